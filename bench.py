"""Benchmark of the FP8 quantized-inference hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

Prints ONE JSON line.  The default workload is the DeepSeek-V3-shaped fused MoE layer, the fifth
configuration of the benchmark definition (hidden 7168, expert intermediate 2048, 256 routed experts, top-8,
one shared expert, T=8192 tokens in total, FP8 weights with 128x128 block scales): the one
configuration of the metric that is defined at 1, 2, 4 and 8 GPUs, so every N reports the same
quantity (tokens/s of the whole layer, strong scaling: the 8192 tokens and 256 experts are
split over the ranks, dispatch/combine over peer memory).  At N=1 the same line also carries the
other half of the metric under "extra": FP8 scaled-mm TFLOP/s on the Llama-3-8B shapes
(second configuration) and block-scaled shapes (third), and act_quant GB/s.

A step = one forward pass of the layer over the step's tokens.  "value" is measured with the
inputs resident in HBM; "e2e" goes through the public layer call with pinned HOST buffers,
host->device copies of the step's activations/router outputs and the device->host read of the
result inside the timed region.  Inputs are synthetic (seeded), weights random-initialised and
quantised as the configuration describes.  Weights (1.4-11.3 GB per rank) exceed the 126 MB
L2, so no explicit L2 flush is needed between iterations.

Every rank runs the same number of steps and collectives: the schedule (warm-up, passes of K
timed steps, end-to-end passes, a fixed tail of steps for the clock sampler) is a function of the
command line only (`step_schedule`), never of what a rank measures.  The reported time is the
median of the passes; every pass is in the JSON line.

--impl reference times the CPU restatement of the reference's algorithm (oracle/) on the host
cores for the same metric on a bounded sample of the same workload: a few experts with ALL the
rows the T=8192 router sends them (so that dequantising an expert's weights is amortised over its
rows as in the full step), scaled to tokens by the rows processed.
"""
import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

HIDDEN, INTER, EXPERTS, TOPK, TOKENS = 7168, 2048, 256, 8, 8192
FP8 = torch.float8_e4m3fn


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"],
                    bf16_tflops_sustained=d.get("bf16_tflops_sustained", d["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


# ---------------------------------------------------------------------------------------------
# synthetic inputs
# ---------------------------------------------------------------------------------------------
def make_router(tokens, experts, topk, seed=0):
    """Zipf(s=1.1) expert popularity over a seeded permutation, Gumbel top-k per token,
    weights = softmax of the selected scores (renormalised), bf16."""
    g = torch.Generator().manual_seed(seed)
    p = torch.arange(1, experts + 1).float() ** -1.1
    p = p[torch.randperm(experts, generator=g)]
    u = torch.rand(tokens, experts, generator=g).clamp_min(1e-9)
    score = torch.log(p / p.sum()) - torch.log(-torch.log(u))
    sc, ids = torch.topk(score, topk)
    return torch.softmax(sc, -1).bfloat16(), ids


def block_quant_weight_gpu(w):
    """[N, K] fp32 on the device -> (fp8 [N, K], fp32 [N/128, K/128]) with 128x128 block scales."""
    n, k = w.shape
    t = w.view(n // 128, 128, k // 128, 128)
    s = t.abs().amax(dim=(1, 3)).clamp_min(1e-10) / torch.tensor(448.0, device=w.device)
    q = (t / s[:, None, :, None]).clamp(-448, 448).view(n, k).to(FP8)
    return q, s


def make_expert_weights(n_experts, first_expert, device, seed=0):
    w1 = torch.empty(n_experts, 2 * INTER, HIDDEN, dtype=FP8, device=device)
    w2 = torch.empty(n_experts, HIDDEN, INTER, dtype=FP8, device=device)
    s1 = torch.empty(n_experts, 2 * INTER // 128, HIDDEN // 128, device=device)
    s2 = torch.empty(n_experts, HIDDEN // 128, INTER // 128, device=device)
    g = torch.Generator(device=device)
    for e in range(n_experts):
        g.manual_seed(seed * 1000003 + first_expert + e)
        w1[e], s1[e] = block_quant_weight_gpu(torch.randn(2 * INTER, HIDDEN, device=device, generator=g) * 0.02)
        w2[e], s2[e] = block_quant_weight_gpu(torch.randn(HIDDEN, INTER, device=device, generator=g) * 0.02)
    return w1, w2, s1, s2


def make_shared_weights(device, seed=0):
    g = torch.Generator(device=device)
    g.manual_seed(seed * 1000003 + 999983)
    a, sa = block_quant_weight_gpu(torch.randn(2 * INTER, HIDDEN, device=device, generator=g) * 0.02)
    b, sb = block_quant_weight_gpu(torch.randn(HIDDEN, INTER, device=device, generator=g) * 0.02)
    return a, b, sa, sb


# ---------------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------------
class ClockSampler:
    """SM clock and throttle reasons of one GPU, sampled in a thread of this process through NVML
    (read-only queries).  NVML is initialised in __enter__, before anything is timed: a freshly
    started `nvidia-smi` process spends its first second enumerating every GPU of the box, and eight
    of them doing so beside the timed passes slowed 8-rank steps by half."""
    REASONS = ((0x8, "hw_slowdown"), (0x40, "hw_thermal_slowdown"), (0x20, "sw_thermal_slowdown"),
               (0x4, "sw_power_cap"))

    def __init__(self, index, interval_ms=100):
        self.index, self.interval = index, max(int(interval_ms), 10) / 1e3
        self.sm, self.reasons_seen, self.max_sm, self.handle, self.nvml = [], 0, None, None, None
        self._stop = threading.Event()
        self.thread = None

    def __enter__(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nvml = pynvml
            try:
                uuid = "GPU-" + str(torch.cuda.get_device_properties(self.index).uuid)
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:  # noqa: BLE001 - fall back to the ordinal
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_sm = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self._sample()
            self.thread = threading.Thread(target=self._run, daemon=True)
            self.thread.start()
        except Exception:  # noqa: BLE001 - no NVML: the clocks record stays empty
            self.nvml = None
        return self

    def _sample(self):
        n = self.nvml
        self.sm.append(float(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)))
        try:
            self.reasons_seen |= int(n.nvmlDeviceGetCurrentClocksEventReasons(self.handle))
        except Exception:  # noqa: BLE001 - older bindings
            self.reasons_seen |= int(n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle))

    def _run(self):
        while not self._stop.wait(self.interval):
            try:
                self._sample()
            except Exception:  # noqa: BLE001
                return

    def __exit__(self, *a):
        self._stop.set()
        if self.thread is not None:
            self.thread.join(timeout=2)
        if self.nvml is not None:
            try:
                self.nvml.nvmlShutdown()
            except Exception:  # noqa: BLE001
                pass

    def summary(self):
        # the first sample was taken before any work was queued; the median is over the rest
        under_load = self.sm[1:] if len(self.sm) > 1 else self.sm
        return {"sm_mhz": statistics.median(under_load) if under_load else None, "sm_max_mhz": self.max_sm,
                "reasons": [name for bit, name in self.REASONS if self.reasons_seen & bit],
                "samples": len(under_load), "source": "NVML, in-process thread"}


# ---------------------------------------------------------------------------------------------
# timing helpers
# ---------------------------------------------------------------------------------------------
def time_events(fn, iters):
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters


def time_graph(fn, iters=10, warm=3, reps=3):
    """Device time of fn per call, launch overhead excluded: `iters` calls captured in one CUDA
    graph and replayed (events on the replay stream)."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    st = torch.cuda.Stream()
    st.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(st):
        with torch.cuda.graph(graph, stream=st):
            for _ in range(iters):
                fn()
    best = None
    for _ in range(reps):
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        graph.replay()
        e.record()
        torch.cuda.synchronize()
        t = s.elapsed_time(e) / iters
        best = t if best is None else min(best, t)
    return best


# ---------------------------------------------------------------------------------------------
# extras at N=1: the dense half of the metric
# ---------------------------------------------------------------------------------------------
def dense_extras(peaks):
    import flag_gems

    out = {"scaled_mm_tflops": {}, "block_scaled_mm_tflops": {}, "quant_gbs": {}}
    fp8_peak = 2.0 * peaks["bf16_tflops"]
    g = torch.Generator(device="cuda")
    g.manual_seed(0)
    # bandwidth kernels first, before the GEMM loops have pushed the part into its power cap
    for (m, kk) in ((256, 4096), (16384, 7168)):
        x = torch.randn(m, kk, device="cuda", generator=g).bfloat16()
        by = m * kk * (2 + 1 + 4 / 128)
        for nm, fn in (("act_quant_g128", lambda: flag_gems.act_quant_triton(x, 128)),
                       ("per_token_group_quant_g128", lambda: flag_gems.per_token_group_quant_fp8(x, 128))):
            ms = time_graph(fn)
            out["quant_gbs"][f"{nm}_M{m}_K{kk}"] = {"gbs": round(by / ms / 1e6, 1), "us": round(ms * 1e3, 1),
                                                   "frac_of_measured_hbm": round(by / ms / 1e6 / peaks["hbm_gbs"], 3)}
    for (name, n, k) in [("qkv", 6144, 4096), ("o", 4096, 4096), ("gate_up", 28672, 4096), ("down", 4096, 14336)]:
        w = (torch.randn(n, k, device="cuda", generator=g) * 0.02)
        sw = w.abs().amax(1).clamp_min(1e-10) / 448.0
        wq = (w / sw[:, None]).clamp(-448, 448).to(FP8)
        del w
        for m in (1, 16, 128, 1024, 4096, 8192):
            a = torch.randn(m, k, device="cuda", generator=g).bfloat16()
            aq, sa = flag_gems.fused.fused_moe._fp8_quantize(a, None, True, None)
            c = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
            ms = time_graph(lambda: flag_gems.cutlass_scaled_mm(c, aq, wq.t(), sa.view(-1), sw))
            tf = 2.0 * m * n * k / ms / 1e9
            by = m * k + n * k + 2 * m * n + 4 * (m + n)
            out["scaled_mm_tflops"][f"{name}_M{m}_N{n}_K{k}"] = {
                "tflops": round(tf, 1), "us": round(ms * 1e3, 1), "frac_of_2x_measured_bf16": round(tf / fp8_peak, 3),
                "frac_of_nominal_4500": round(tf / 4500.0, 3),
                "frac_of_measured_hbm": round(by / ms / 1e6 / peaks["hbm_gbs"], 3)}
    k = 7168
    for n in (2112, 4096, 18432, 24576):
        w = torch.randn((n + 127) // 128 * 128, k, device="cuda", generator=g) * 0.02
        wq, ws = block_quant_weight_gpu(w)
        wq = wq[:n].contiguous()
        del w
        for m in (1, 64, 512, 4096, 16384):
            a = torch.randn(m, k, device="cuda", generator=g).bfloat16()
            aq, a_s = flag_gems.per_token_group_quant_fp8(a, 128)
            ms = time_graph(lambda: flag_gems.w8a8_block_fp8_matmul(aq, wq, a_s, ws, [128, 128]), iters=5)
            tf = 2.0 * m * n * k / ms / 1e9
            by = m * k + n * k + 2 * m * n + 4 * m * (k // 128) + 4 * ((n + 127) // 128) * (k // 128)
            out["block_scaled_mm_tflops"][f"M{m}_N{n}_K{k}"] = {
                "tflops": round(tf, 1), "us": round(ms * 1e3, 1), "frac_of_2x_measured_bf16": round(tf / fp8_peak, 3),
                "frac_of_nominal_4500": round(tf / 4500.0, 3),
                "frac_of_measured_hbm": round(by / ms / 1e6 / peaks["hbm_gbs"], 3)}
    ids = make_router(TOKENS, EXPERTS, TOPK)[1].cuda()
    ms = time_graph(lambda: flag_gems.moe_align_block_size(ids, 64, EXPERTS), iters=20)
    out["moe_align_us"] = {"T8192_top8_E256_bs64": round(ms * 1e3, 1)}
    ids4 = torch.topk(torch.softmax(torch.randn(4096, 8, generator=torch.Generator().manual_seed(0)), -1), 2)[1].cuda()
    ms = time_graph(lambda: flag_gems.moe_align_block_size(ids4, 64, 8), iters=20)
    out["moe_align_us"]["T4096_top2_E8_bs64"] = round(ms * 1e3, 1)

    # router kernels in front of the layer (DeepSeek-V3 routing shape): device time and HBM fraction
    logits = torch.randn(TOKENS, EXPERTS, device="cuda", generator=g)
    rbias = torch.randn(EXPERTS, device="cuda", generator=g) * 0.1
    rw = torch.empty(TOKENS, TOPK, device="cuda")
    ri = torch.empty(TOKENS, TOPK, dtype=torch.int32, device="cuda")
    rs = torch.empty(TOKENS, TOPK, dtype=torch.int32, device="cuda")
    router_bytes = TOKENS * EXPERTS * 4 + TOKENS * TOPK * 12
    ms = time_graph(lambda: flag_gems.topk_softmax(rw, ri, rs, logits, True), iters=20)
    out["router_us"] = {"topk_softmax_T8192_E256_top8": round(ms * 1e3, 1),
                        "topk_softmax_gbs": round(router_bytes / ms / 1e6, 1)}
    ms = time_graph(lambda: flag_gems.grouped_topk(logits, 8, 4, TOPK, True, 2.5, rbias, 1), iters=20)
    out["router_us"]["grouped_topk_T8192_E256_g8_tg4_top8_sigmoid"] = round(ms * 1e3, 1)
    out["router_us"]["grouped_topk_gbs"] = round((router_bytes - TOKENS * TOPK * 4) / ms / 1e6, 1)

    # fourth benchmark configuration: Mixtral-8x7B-shaped layer, per-token x per-channel FP8, through fused_experts_impl
    t4, h4, i4, e4 = 4096, 4096, 14336, 8
    w1 = torch.empty(e4, 2 * i4, h4, dtype=FP8, device="cuda")
    w2 = torch.empty(e4, h4, i4, dtype=FP8, device="cuda")
    s1 = torch.empty(e4, 2 * i4, device="cuda")
    s2 = torch.empty(e4, h4, device="cuda")
    for e in range(e4):
        for (wq, sq, shape) in ((w1, s1, (2 * i4, h4)), (w2, s2, (h4, i4))):
            w = torch.randn(*shape, device="cuda", generator=g) * 0.02
            sc = w.abs().amax(1).clamp_min(1e-10) / 448.0
            wq[e], sq[e] = (w / sc[:, None]).clamp(-448, 448).to(FP8), sc
            del w
    hid = torch.randn(t4, h4, device="cuda", generator=g).bfloat16()
    tw4, ti4 = torch.topk(torch.softmax(torch.randn(t4, e4, device="cuda", generator=g), -1), 2)
    tw4 = (tw4 / tw4.sum(-1, keepdim=True)).bfloat16()
    fn = lambda: flag_gems.fused_experts_impl(hid, w1, w2, tw4, ti4, use_fp8_w8a8=True, per_channel_quant=True,
                                              w1_scale=s1, w2_scale=s2)
    for _ in range(3):
        fn()
    ms = time_events(fn, 10)
    out["moe_mixtral_8x7b"] = {"tokens_per_s": round(t4 / ms * 1e3, 1), "ms": round(ms, 3),
                               "tflops": round(2.0 * t4 * 2 * 3 * h4 * i4 / ms / 1e9, 1),
                               "config": "T=4096, hidden 4096, intermediate 14336, 8 experts, top-2, "
                                         "per-token x per-channel FP8 (configs[3]), fused_experts_impl"}
    # the same layer with int8 w8a8 experts (per-token x per-channel), tcgen05 kind::i8
    s1i, s2i = s1 * (448.0 / 127.0), s2 * (448.0 / 127.0)
    w1i = (w1.float() * (127.0 / 448.0)).round().clamp(-127, 127).to(torch.int8)
    w2i = (w2.float() * (127.0 / 448.0)).round().clamp(-127, 127).to(torch.int8)
    del w1, w2
    fn = lambda: flag_gems.fused_experts_impl(hid, w1i, w2i, tw4, ti4, use_int8_w8a8=True, per_channel_quant=True,
                                              w1_scale=s1i, w2_scale=s2i)
    for _ in range(3):
        fn()
    ms = time_events(fn, 10)
    out["moe_mixtral_8x7b_int8"] = {"tokens_per_s": round(t4 / ms * 1e3, 1), "ms": round(ms, 3),
                                    "tops": round(2.0 * t4 * 2 * 3 * h4 * i4 / ms / 1e9, 1)}
    # and unquantised bf16 experts (the default path of fused_experts_impl), tcgen05 kind::f16
    w1b, w2b = w1i.bfloat16() * 0.01, w2i.bfloat16() * 0.01
    del w1i, w2i
    fn = lambda: flag_gems.fused_experts_impl(hid, w1b, w2b, tw4, ti4)
    for _ in range(3):
        fn()
    ms = time_events(fn, 10)
    out["moe_mixtral_8x7b_bf16"] = {"tokens_per_s": round(t4 / ms * 1e3, 1), "ms": round(ms, 3),
                                    "tflops": round(2.0 * t4 * 2 * 3 * h4 * i4 / ms / 1e9, 1)}
    del w1b, w2b

    # aten _scaled_grouped_mm (rows of A grouped by device-side offsets, one B per group), expert-GEMM shaped
    gg, mg, ng, kg = 32, 8192, 4096, 7168
    ag = torch.randn(mg, kg, device="cuda", generator=g).to(FP8)
    bg = torch.randn(gg, ng, kg, device="cuda", generator=g).to(FP8)
    sag = torch.rand(mg, device="cuda") + 0.5
    sbg = torch.rand(gg, ng, device="cuda") + 0.5
    offs = (torch.arange(1, gg + 1, device="cuda", dtype=torch.int32) * (mg // gg))
    fn = lambda: flag_gems.scaled_grouped_mm(ag, bg.transpose(-1, -2), sag, sbg, offs)
    ms = time_graph(fn, iters=10)
    out["scaled_grouped_mm_tflops"] = {f"G{gg}_M{mg}_N{ng}_K{kg}": {"tflops": round(2.0 * mg * ng * kg / ms / 1e9, 1),
                                                                    "us": round(ms * 1e3, 1)}}
    del ag, bg

    # The vendor library's FP8 GEMM under the same conditions, for scale (cuBLASLt via torch._scaled_mm).
    try:
        m = n = k = 8192
        a = torch.randn(m, k, device="cuda", generator=g).to(FP8)
        b = torch.randn(n, k, device="cuda", generator=g).to(FP8)
        one = torch.ones((), device="cuda")
        sa, sb = torch.rand(m, 1, device="cuda") + 0.5, torch.rand(1, n, device="cuda") + 0.5
        c = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
        lib = {}
        ms = time_graph(lambda: torch._scaled_mm(a, b.t(), one, one, out_dtype=torch.bfloat16), iters=5)
        lib["cublaslt_tensorwise_8192"] = round(2.0 * m * n * k / ms / 1e9, 1)
        ms = time_graph(lambda: torch._scaled_mm(a, b.t(), sa, sb, out_dtype=torch.bfloat16), iters=5)
        lib["cublaslt_rowwise_8192"] = round(2.0 * m * n * k / ms / 1e9, 1)
        ms = time_graph(lambda: flag_gems.cutlass_scaled_mm(c, a, b.t(), sa.view(-1), sb.view(-1)), iters=5)
        lib["this_library_rowwise_8192"] = round(2.0 * m * n * k / ms / 1e9, 1)
        out["library_fp8_tflops"] = lib
    except Exception as exc:  # noqa: BLE001 - comparison only
        out["library_fp8_tflops"] = {"unavailable": str(exc)[:200]}
    return out


# ---------------------------------------------------------------------------------------------
# CPU arm (oracle)
# ---------------------------------------------------------------------------------------------
def cpu_expert_sample(experts, rows_of, fetch_expert, shared, hidden_of):
    """The oracle's layer restricted to `experts`, each with ALL the rows routed to it, plus the
    shared expert on as many tokens as those rows amount to (rows / top-k).
    rows_of(e) -> (token indices, router weights); fetch_expert(e) -> (w1, w2, s1, s2) CPU tensors;
    hidden_of(tokens) -> [n, H] bf16.  Returns ({e: rows' results}, seconds, rows processed)."""
    import oracle

    results, n_rows, dt = {}, 0, 0.0
    for e in experts:
        tok, wts = rows_of(e)
        if tok.numel() == 0:
            continue
        w = fetch_expert(e)
        x = hidden_of(tok)
        t0 = time.perf_counter()
        results[e] = oracle.expert_rows_block_fp8(x, *w, wts)
        dt += time.perf_counter() - t0
        n_rows += tok.numel()
    n_tok = max(1, n_rows // TOPK)
    x = hidden_of(torch.arange(n_tok))
    t0 = time.perf_counter()
    oracle.dense_block_fp8_mlp(x, *shared)
    dt += time.perf_counter() - t0
    return results, dt, n_rows


def sample_experts(ti, n=4):
    """A fixed, routing-derived choice of experts for the CPU legs: the busiest expert, the one with
    the fewest (non-zero) rows, and n - 2 around the median, by routed-row count."""
    counts = torch.bincount(ti.reshape(-1), minlength=EXPERTS)
    order = torch.argsort(counts, descending=True, stable=True).tolist()
    order = [e for e in order if counts[e] > 0]
    mid = len(order) // 2
    picks = [order[0], order[-1]] + order[mid:mid + max(0, n - 2)]
    return sorted(set(picks)), counts


def cpu_weight_pool(pool=4, seed=0):
    import oracle

    g = torch.Generator().manual_seed(seed)
    sets = []
    for _ in range(pool):
        w1, s1 = oracle.quantize_weight_block(torch.randn(2 * INTER, HIDDEN, generator=g) * 0.02)
        w2, s2 = oracle.quantize_weight_block(torch.randn(HIDDEN, INTER, generator=g) * 0.02)
        sets.append((w1, w2, s1, s2))
    return sets


def run_reference(args):
    """CPU arm: the oracle on all host threads; each step = two experts with all their routed rows."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    pool = cpu_weight_pool()
    shared = pool[0]
    tw, ti = make_router(TOKENS, EXPERTS, TOPK)
    counts = torch.bincount(ti.reshape(-1), minlength=EXPERTS)
    order = torch.argsort(counts, descending=True, stable=True).tolist()
    mid = len(order) // 2  # experts around the median load: ~T*topk/E rows each
    g = torch.Generator().manual_seed(1)
    hidden = torch.randn(TOKENS, HIDDEN, generator=g).bfloat16()

    def rows_of(e):
        tok, slot = torch.nonzero(ti == e, as_tuple=True)
        return tok, tw[tok, slot]

    times, rows_done = [], []
    for step in range(args.warmup + args.steps):
        experts = [order[(mid + 2 * step) % len(order)], order[(mid + 2 * step + 1) % len(order)]]
        _, dt, n_rows = cpu_expert_sample(experts, rows_of, lambda e: pool[e % len(pool)], shared,
                                          lambda tok: hidden[tok])
        if step >= args.warmup:
            times.append(dt)
            rows_done.append(n_rows)
    tokens_equiv = sum(rows_done) / TOPK
    total = sum(times)
    value = tokens_equiv / total
    ms = 1e3 * total / len(times)
    desc = (f"per step two experts of median load with ALL rows the T={TOKENS} router sends them "
            f"({sum(rows_done) / len(rows_done):.0f} rows per step on average) plus the shared expert on rows/top-{TOPK} "
            f"tokens; tokens = rows / {TOPK}; expert weights from a pool of {len(pool)} generated sets; "
            f"oracle/ torch-CPU fp32")
    line = {
        "impl": "reference", "metric": "fused_moe_tokens_per_s", "value": round(value, 3), "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 3),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp8_e4m3",
        "data": "synthetic", "config": workload_config(args.gpus),
        "cpu_baseline": {"value": round(value, 3), "unit": "tokens/s", "cores": torch.get_num_threads(),
                         "kind": "port", "sample": desc},
        "e2e": {"value": round(value, 3), "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(n):
    return {"workload": "deepseek_v3_moe_layer (configs[4])", "hidden": HIDDEN, "intermediate": INTER,
            "experts": EXPERTS, "top_k": TOPK, "shared_experts": 1, "tokens_global": TOKENS,
            "weight_format": "fp8_e4m3 128x128 block scales", "activation_format": "fp8_e4m3 1x128 group scales",
            "router": "zipf(1.1) gumbel top-8, seed 0", "parallelism": f"ep{n}",
            "expert_placement": "static, load-balanced over ranks from the routing counts (greedy longest-first)",
            "l2": "weights per rank (>=1.4 GB) exceed L2; no explicit flush"}


# ---------------------------------------------------------------------------------------------
# main arm
# ---------------------------------------------------------------------------------------------
CLOCK_TAIL_STEPS = 200  # resident steps after the timed passes, so the clock sampler sees load


def step_schedule(args):
    """What every rank runs, in order, as (phase, number of steps).  A function of the command
    line only: ranks must issue identical sequences of collectives, so nothing a rank observes
    (time, clock samples, its own load) may change how many steps it runs."""
    warm = max(args.warmup, 3)
    sched = [("warmup", warm)]
    sched += [("timed", args.steps)] * args.passes
    sched += [("e2e_warmup", 2)]
    sched += [("e2e", args.steps)] * args.passes
    sched += [("clock_tail", CLOCK_TAIL_STEPS), ("phase_trace", 1)]
    return sched


def run_ours(args):
    import datetime

    import torch.distributed as dist

    import flag_gems  # noqa: F401
    from flaggems_b200 import _cabi
    from flaggems_b200.ep import ExpertParallelMoE, balanced_expert_placement

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback "
                         "(use --impl reference for the CPU arm)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # a short timeout: ranks whose collectives stop matching give up within a minute
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=60))
    assert world == args.gpus or world == 1, f"WORLD_SIZE {world} != --gpus {args.gpus}"
    layer = None
    try:
        layer = _run_ours(args, world, rank, local_rank, dev, dist, _cabi, ExpertParallelMoE,
                          balanced_expert_placement)
    finally:
        # ordered teardown: graphs, device idle, barrier, peer mappings, buffers; then the group
        if layer is not None:
            layer.close()
        if world > 1:
            dist.destroy_process_group()


def _run_ours(args, world, rank, local_rank, dev, dist, _cabi, ExpertParallelMoE, balanced_expert_placement):
    peaks = load_peaks()
    e_loc, t_loc = EXPERTS // world, TOKENS // world
    w1, w2, s1, s2 = make_expert_weights(e_loc, rank * e_loc, dev)
    shared = make_shared_weights(dev)
    transport = "a2a" if args.a2a_combine else ("p2p_combine" if args.a2a_dispatch else "p2p")
    layer = ExpertParallelMoE(w1, w2, s1, s2, EXPERTS, rank, world, shared=shared, transport=transport,
                              max_slots_per_rank=t_loc * TOPK)
    tw_all, ti_all = make_router(TOKENS, EXPERTS, TOPK)
    # logical expert -> physical slot (rank * E_loc + local index); identical on every rank
    placement = balanced_expert_placement(torch.bincount(ti_all.reshape(-1), minlength=EXPERTS), world)
    ti_all = placement[ti_all]
    rows_per_rank = torch.bincount((ti_all // e_loc).reshape(-1), minlength=world)
    sl = slice(rank * t_loc, (rank + 1) * t_loc)
    g = torch.Generator().manual_seed(100 + rank)
    hidden_h = torch.randn(t_loc, HIDDEN, generator=g).bfloat16().pin_memory()
    tw_h, ti_h = tw_all[sl].contiguous().pin_memory(), ti_all[sl].contiguous().pin_memory()
    out_h = torch.empty(t_loc, HIDDEN, dtype=torch.bfloat16).pin_memory()
    hidden_d, tw_d, ti_d = hidden_h.to(dev), tw_h.to(dev), ti_h.to(dev)

    # The step is recorded once into a CUDA graph and replayed (same kernels, collectives and
    # streams as the eager call, one host launch per step) unless an all-to-all transport, which
    # waits on the host for its counts, or --no-graph is chosen.
    use_graph = (not args.no_graph) and (world == 1 or transport == "p2p")
    if use_graph:
        layer.capture(hidden_d, tw_d, ti_d)

        def step_resident():
            return layer.replay()

        # End to end as a serving loop runs it: the host->device copy of step k+1's inputs and the
        # device->host copy of step k-1's result ride on their own streams beside step k's kernels
        # (double-buffered staging on the device; every step still pays both copies in full).
        st_h2d, st_d2h = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        stage_in = [(torch.empty_like(hidden_d), torch.empty_like(tw_d), torch.empty_like(ti_d)) for _ in range(2)]
        stage_out = [torch.empty(t_loc, HIDDEN, dtype=torch.bfloat16, device=dev) for _ in range(2)]
        out_hs = [out_h, torch.empty_like(out_h).pin_memory()]
        ev_staged = [torch.cuda.Event() for _ in range(2)]
        ev_in_free = [torch.cuda.Event() for _ in range(2)]
        ev_out = [torch.cuda.Event() for _ in range(2)]
        ev_out_free = [torch.cuda.Event() for _ in range(2)]
        e2e_k = [0]

        def step_e2e():
            k = e2e_k[0]
            e2e_k[0] += 1
            b = k & 1
            main = torch.cuda.current_stream(dev)
            with torch.cuda.stream(st_h2d):
                if k >= 2:
                    st_h2d.wait_event(ev_in_free[b])
                for dst, src in zip(stage_in[b], (hidden_h, tw_h, ti_h)):
                    dst.copy_(src, non_blocking=True)
                ev_staged[b].record(st_h2d)
            main.wait_event(ev_staged[b])
            for dst, src in zip((hidden_d, tw_d, ti_d), stage_in[b]):
                dst.copy_(src, non_blocking=True)
            ev_in_free[b].record(main)
            out = layer.replay()
            if k >= 2:
                main.wait_event(ev_out_free[b])
            stage_out[b].copy_(out, non_blocking=True)
            ev_out[b].record(main)
            with torch.cuda.stream(st_d2h):
                st_d2h.wait_event(ev_out[b])
                out_hs[b].copy_(stage_out[b], non_blocking=True)
                ev_out_free[b].record(st_d2h)
    else:
        def step_resident():
            return layer(hidden_d, tw_d, ti_d)

        def step_e2e():
            h = hidden_h.to(dev, non_blocking=True)
            w = tw_h.to(dev, non_blocking=True)
            i = ti_h.to(dev, non_blocking=True)
            out_h.copy_(layer(h, w, i), non_blocking=True)
            torch.cuda.current_stream().synchronize()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    extra_streams = []

    def timed(fn, steps):
        barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(steps):
            fn()
        for st in extra_streams:  # copies still in flight on the side streams belong to the region
            torch.cuda.current_stream().wait_stream(st)
        e.record()
        torch.cuda.synchronize()
        ms = s.elapsed_time(e) / steps
        barrier()
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    # Clocks are sampled from the first warm-up step to the end of the schedule: the same
    # workload throughout, long enough for nvidia-smi to report whatever the step time is.
    ms_passes, e2e_passes, marks = [], [], []
    launches0 = launches = 0
    with ClockSampler(local_rank, args.clock_interval_ms) as clocks:
        for phase, n in step_schedule(args):
            if phase in ("warmup", "clock_tail"):
                for _ in range(n):
                    step_resident()
                if phase == "warmup":
                    launches0 = _cabi.launch_count()
            elif phase == "timed":
                ms_passes.append(timed(step_resident, n))
                launches = _cabi.launch_count() - launches0
            elif phase == "e2e_warmup":
                for _ in range(n):
                    step_e2e()
                if use_graph:
                    extra_streams.extend([st_h2d, st_d2h])
            elif phase == "e2e":
                e2e_passes.append(timed(step_e2e, n))
            elif phase == "phase_trace":
                del extra_streams[:]
                barrier()
                # phase breakdown of one eager step on this rank (CUDA events on the layer's stream);
                # the first eager step after the graph replays re-warms the eager path untimed
                layer(hidden_d, tw_d, ti_d)
                torch.cuda.synchronize()
                layer.trace = []
                layer(hidden_d, tw_d, ti_d)
                torch.cuda.synchronize()
                marks, layer.trace = layer.trace, None
        torch.cuda.synchronize()
    ms = statistics.median(ms_passes)
    ms_e2e = statistics.median(e2e_passes)
    launches = launches // args.passes
    if use_graph:
        launches = layer.kernels_per_replay * args.steps
    phases = {marks[i][0]: round(marks[i - 1][1].elapsed_time(marks[i][1]), 4) for i in range(1, len(marks))}
    status = _cabi.device_status()
    barrier()  # from here on no rank issues a collective until close()

    # dominant kernel: the grouped GEMM1 (block-scaled, fused SiLU) on this rank's routed rows,
    # timed alone on the launching stream with CUDA events.
    from flaggems_b200.fused.fused_moe import _TILE_ROWS, _group_quant, _grouped_gemm
    from flaggems_b200.fused.moe_align_block_size import moe_align_block_size

    if world == 1:
        ids_local, n_rows, hid_src, div = ti_d, t_loc * TOPK, hidden_d, TOPK
    else:
        # rows this rank's experts receive: recompute the global routing (identical on every rank)
        owner = ti_all // e_loc
        mask = owner == rank
        n_rows = int(mask.sum())
        ids_local = (ti_all[mask] % e_loc).to(torch.int32).to(dev)
        hid_src, div = torch.randn(n_rows, HIDDEN, device=dev).bfloat16(), 1
    sorted_ids, expert_ids, post_pad = moe_align_block_size(ids_local, _TILE_ROWS, e_loc)
    rows = sorted_ids.numel() // _TILE_ROWS * _TILE_ROWS
    a1, a1s = _group_quant(hid_src, 128, sorted_ids, div, n_rows, post_pad, rows)
    act = torch.empty((rows, INTER), dtype=torch.bfloat16, device=dev)

    def gemm1():
        _grouped_gemm(act, a1, w1, a1s, layer.ops.w1_scale, None, sorted_ids, expert_ids, post_pad, n_rows,
                      _cabi.SCALE_BLOCK, fuse_silu=True, scatter=False, mul_weight=False)

    for _ in range(3):
        gemm1()
    gemm1_ms = time_events(gemm1, max(args.steps, 5))
    gemm1_flops = 2.0 * n_rows * (2 * INTER) * HIDDEN
    achieved = gemm1_flops / gemm1_ms / 1e9
    fp8_peak = 2.0 * peaks["bf16_tflops_sustained"]
    roofline = {"bound": "tensor", "kernel": "gemm_fp8_kernel<BN, block_scaled, fuse_silu> (MoE GEMM1)",
                "achieved": round(achieved, 1), "peak": round(fp8_peak, 1), "unit": "TFLOP/s",
                "frac": round(achieved / fp8_peak, 4),
                # dram__bytes_read + write of this kernel from an ncu capture of a 32-expert / 8192-row
                # case (one eighth of the single-GPU launch), scaled by the experts held by this rank
                "traffic": round(1.2031e9 * e_loc / 32),
                "hbm_gbs_at_that_traffic": round(1.2031e9 * e_loc / 32 / gemm1_ms / 1e6, 1),
                "peak_source": f"2 x {peaks['source']} sustained dense bf16 cuBLAS TF/s (fp8 tensor rate is twice bf16)",
                "frac_of_2x_measured_bf16_burst": round(achieved / (2.0 * peaks["bf16_tflops"]), 4),
                "frac_of_nominal_4500": round(achieved / 4500.0, 4), "launch_ms": round(gemm1_ms, 4),
                "algorithmic_flops_per_launch": gemm1_flops, "rows": n_rows}

    value = TOKENS / (ms / 1e3)
    e2e_value = TOKENS / (ms_e2e / 1e3)
    h2d = hidden_h.numel() * 2 + tw_h.numel() * 2 + ti_h.numel() * 8
    d2h_bytes = out_h.numel() * 2
    line = {
        "metric": "fused_moe_tokens_per_s", "value": round(value, 1), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "fp8_e4m3", "data": "synthetic",
        "config": workload_config(world), "clocks": clocks.summary(),
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d * world,
                "d2h_bytes_per_step": d2h_bytes * world, "ms_per_step": round(ms_e2e, 4),
                "copies": ("pinned host buffers; the copies of neighbouring steps overlap the kernels on their own "
                           "streams (double-buffered)" if use_graph else "pinned host buffers, serial with the kernels")},
        "gpu_launches": int(launches), "roofline": roofline, "device_status": status,
        "launch_mode": "CUDA graph replay (step recorded once)" if use_graph else "eager",
        "timing": {"passes_of_k_steps": args.passes, "reported": "median pass",
                   "ms_per_step_passes": [round(x, 4) for x in ms_passes],
                   "e2e_ms_per_step_passes": [round(x, 4) for x in e2e_passes]},
        "phase_ms_rank0_eager_step": phases,
        "dispatch": ("n/a (single rank)" if world == 1 else
                     "NCCL all_to_all_single" if transport != "p2p" else
                     "fused into the quantisation kernel: packed rows stored into this rank's region of the "
                     "destination's receive buffer over NVLink peer memory; counts by a stream-ordered all-gather "
                     "that doubles as the arrival barrier (no host wait in the step)"),
        "combine": ("n/a (single rank)" if world == 1 else
                    "NCCL all_to_all_single" if transport == "a2a" else
                    "fused into GEMM2's epilogue: rows stored to the home rank over NVLink peer memory"),
        "collectives_per_step": 0 if world == 1 else (2 if transport == "p2p" else 3 if transport == "p2p_combine" else 4),
        "routed_rows_per_rank": {"max": int(rows_per_rank.max()), "mean": float(rows_per_rank.float().mean())},
        "layer_tflops": round((2.0 * TOKENS * TOPK * 3 * HIDDEN * INTER + 2.0 * TOKENS * 3 * HIDDEN * INTER) / ms / 1e9, 1),
    }

    if rank == 0 and world == 1:
        line.update(cpu_legs_single_gpu(args, layer, hidden_d, tw_d, ti_d, hidden_h, tw_h, ti_h, w1, w2, s1, s2,
                                        shared))
        if not args.no_extras:
            line["extra"] = dense_extras(peaks)
    if rank == 0:
        print(json.dumps(line), flush=True)
    return layer


def cpu_legs_single_gpu(args, layer, hidden_d, tw_d, ti_d, hidden_h, tw_h, ti_h, w1, w2, s1, s2, shared):
    """CPU baseline and full-size parity at N=1, on the step's own tensors and weights (copied from
    the device).  Parity is checked where the oracle can afford it at T=8192: (a) every row routed
    to a few experts (busiest, emptiest, median ones), per row and per element, through
    quantisation -> GEMM1 -> SiLU -> quantisation -> GEMM2 -> router weight; (b) the layer's final
    output (top-k sum + shared expert) on the first --cpu-tokens tokens."""
    import oracle
    from flaggems_b200 import _cabi

    torch.set_num_threads(os.cpu_count() or 1)
    out = {}
    routed = layer.ops.local_routed(hidden_d, ti_d, tw_d)  # [T*topk, H] bf16 in route-slot order
    out_d = layer(hidden_d, tw_d, ti_d)
    torch.cuda.synchronize()
    experts, counts = sample_experts(ti_h, args.cpu_experts)

    def rows_of(e):
        tok, slot = torch.nonzero(ti_h == e, as_tuple=True)
        return tok, tw_h[tok, slot]

    def fetch(e):
        return w1[e].cpu(), w2[e].cpu(), s1[e].cpu(), s2[e].cpu()

    shared_cpu = tuple(t.cpu() for t in shared)
    results, dt, n_rows = cpu_expert_sample(experts, rows_of, fetch, shared_cpu, lambda tok: hidden_h[tok])
    out["cpu_baseline"] = {
        "value": round(n_rows / TOPK / dt, 3), "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
        "sample": (f"experts {experts} of the step (busiest, emptiest, median load) with ALL {n_rows} rows routed to "
                   f"them, plus the shared expert on rows/top-{TOPK} tokens, same weights; tokens = rows / {TOPK}; "
                   f"oracle/ torch-CPU fp32, {dt:.1f} s")}
    worst, n_el, n_ok = 0.0, 0, 0
    for e, ref in results.items():
        tok, slot = torch.nonzero(ti_h == e, as_tuple=True)
        got = routed[(tok * TOPK + slot).to(routed.device)].cpu().float()
        err = (got - ref.float()).abs()
        tol = 1e-2 + 1e-2 * ref.float().abs()
        worst = max(worst, float((err - tol).max()))
        n_el += err.numel()
        n_ok += int((err <= tol).sum())
    n = args.cpu_tokens
    add = oracle.dense_block_fp8_mlp(hidden_h[:n].clone(), *shared_cpu)
    touched = sorted(set(ti_h[:n].reshape(-1).tolist()))
    remap = {e: i for i, e in enumerate(touched)}
    ws = [fetch(e) for e in touched]
    ref = oracle.fused_moe_block_fp8(hidden_h[:n].clone(), torch.stack([w[0] for w in ws]), torch.stack([w[1] for w in ws]),
                                     torch.stack([w[2] for w in ws]), torch.stack([w[3] for w in ws]), tw_h[:n].clone(),
                                     ti_h[:n].clone().apply_(lambda e: remap[e]), addend=add)
    err = (out_d[:n].cpu().float() - ref.float()).abs()
    tol = 1e-2 + 1e-2 * ref.float().abs()
    # Rows are rounded to bf16 before the fp32 top-k sum (as in the reference), so one bf16 ulp of
    # the largest addend can survive cancellation in the FINAL output: there the strict elementwise
    # bound holds for all but a few elements and the bound relative to max|ref| for all.  The
    # per-row results before the sum have no such cancellation and meet the strict bound.
    out["parity_sample"] = {
        "routed_rows": {"experts": experts, "rows": n_rows, "elements": n_el,
                        "frac_within_rtol1e-2_atol1e-2": n_ok / max(n_el, 1),
                        "worst_excess_over_bound": worst},
        "final_output": {"tokens": n, "max_abs_err": float(err.max()), "max_abs_ref": float(ref.float().abs().max()),
                         "frac_within_rtol1e-2_atol1e-2": float((err <= tol).float().mean()),
                         "all_within_rtol1e-2_atol_1e-2_of_max": bool(
                             (err <= 1e-2 * ref.float().abs() + max(1e-2, 1e-2 * float(ref.float().abs().max()))).all())}}
    assert _cabi.device_status() == 0
    return out


# ---------------------------------------------------------------------------------------------
# small single-kernel cases for profiler captures (not benchmark lines)
# ---------------------------------------------------------------------------------------------
def run_capture_case(args):
    """A few launches of ONE kernel on a case small enough for a profiler capture (inputs larger than
    L2, at most a few GB on the device).  Prints a JSON line marked "capture_case": never a bench value.
      moe_gemm1    grouped block-scaled GEMM1 with fused SiLU, 32 experts / the rows the T=8192 router sends
                   them (one rank's share at 8 ranks; an eighth of the single-GPU launch)
      moe_gemm2    the matching GEMM2 (router weight, rows scattered back)
      moe_gemm1_bf16  GEMM1 of the same shape on unquantised bf16 operands
      block_mm     w8a8 block-scaled GEMM, M = N = 8192, K = 7168
      scaled_mm    per-token x per-channel GEMM, same shape
      group_quant  per_token_group_quant_fp8 and act_quant on [16384, 7168] bf16
      moe_glue     the FP8 row gather into expert order and the top-k sum, on 2048 tokens of the layer"""
    import flag_gems
    from flaggems_b200 import _cabi
    from flaggems_b200.fused.fused_moe import _TILE_ROWS, _group_quant, _grouped_gemm
    from flaggems_b200.fused.moe_align_block_size import moe_align_block_size

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator(device=dev)
    g.manual_seed(0)
    name, n_launch = args.workload, max(1, args.steps)
    if name in ("moe_gemm1", "moe_gemm2"):
        e = 32
        w1, w2, s1, s2 = make_expert_weights(e, 0, dev)
        from flaggems_b200.ep import balanced_expert_placement

        _, ti = make_router(TOKENS, EXPERTS, TOPK)
        ti = balanced_expert_placement(torch.bincount(ti.reshape(-1), minlength=EXPERTS), EXPERTS // e)[ti]
        ids = ti[ti < e].to(torch.int32).to(dev)  # the experts rank 0 holds at 8 ranks
        n_rows = ids.numel()
        hid = torch.randn(n_rows, HIDDEN, device=dev, generator=g).bfloat16()
        sorted_ids, expert_ids, post_pad = moe_align_block_size(ids, _TILE_ROWS, e)
        rows = sorted_ids.numel() // _TILE_ROWS * _TILE_ROWS
        a1, a1s = _group_quant(hid, 128, sorted_ids, 1, n_rows, post_pad, rows)
        act = torch.empty((rows, INTER), dtype=torch.bfloat16, device=dev)

        def gemm1():
            _grouped_gemm(act, a1, w1, a1s, s1.float().contiguous(), None, sorted_ids, expert_ids, post_pad, n_rows,
                          _cabi.SCALE_BLOCK, fuse_silu=True, scatter=False, mul_weight=False)

        gemm1()
        a2, a2s = _group_quant(act, 128, None, 1, 0, post_pad, rows)
        out = torch.empty((n_rows, HIDDEN), dtype=torch.bfloat16, device=dev)
        wts = torch.rand(n_rows, device=dev, generator=g).bfloat16()

        def gemm2():
            _grouped_gemm(out, a2, w2, a2s, s2.float().contiguous(), wts, sorted_ids, expert_ids, post_pad, n_rows,
                          _cabi.SCALE_BLOCK, fuse_silu=False, scatter=True, mul_weight=True)

        fn = gemm1 if name == "moe_gemm1" else gemm2
        flops = 2.0 * n_rows * (2 * INTER if name == "moe_gemm1" else HIDDEN) * (HIDDEN if name == "moe_gemm1" else INTER)
        info = {"experts": e, "rows": n_rows, "rows_padded": int(post_pad)}
    elif name == "moe_gemm1_bf16":
        # the same grouped GEMM1 on unquantised bf16 operands (tcgen05 kind::f16)
        from flaggems_b200.ep import balanced_expert_placement

        e = 32
        _, ti = make_router(TOKENS, EXPERTS, TOPK)
        ti = balanced_expert_placement(torch.bincount(ti.reshape(-1), minlength=EXPERTS), EXPERTS // e)[ti]
        ids = ti[ti < e].to(torch.int32).to(dev)
        n_rows = ids.numel()
        sorted_ids, expert_ids, post_pad = moe_align_block_size(ids, _TILE_ROWS, e)
        rows = sorted_ids.numel() // _TILE_ROWS * _TILE_ROWS
        a1 = torch.randn(rows, HIDDEN, device=dev, generator=g).bfloat16()
        w1 = (torch.randn(e, 2 * INTER, HIDDEN, device=dev, generator=g) * 0.02).bfloat16()
        act = torch.empty((rows, INTER), dtype=torch.bfloat16, device=dev)
        one_a = torch.ones(1, device=dev)
        one_b = torch.ones(e, device=dev)

        def fn():
            _grouped_gemm(act, a1, w1, one_a, one_b, None, sorted_ids, expert_ids, post_pad, n_rows,
                          _cabi.SCALE_SCALAR, fuse_silu=True, scatter=False, mul_weight=False)

        flops = 2.0 * n_rows * 2 * INTER * HIDDEN
        info = {"experts": e, "rows": n_rows, "rows_padded": int(post_pad)}
    elif name in ("block_mm", "scaled_mm"):
        m = n = 8192
        k = 7168
        a = torch.randn(m, k, device=dev, generator=g).bfloat16()
        w = torch.randn(n, k, device=dev, generator=g) * 0.02
        if name == "block_mm":
            aq, a_s = flag_gems.per_token_group_quant_fp8(a, 128)
            wq, ws = block_quant_weight_gpu(w)
            fn = lambda: flag_gems.w8a8_block_fp8_matmul(aq, wq, a_s, ws, [128, 128])  # noqa: E731
        else:
            aq, sa = flag_gems.fused.fused_moe._fp8_quantize(a, None, True, None)
            sw = w.abs().amax(1).clamp_min(1e-10) / 448.0
            wq = (w / sw[:, None]).clamp(-448, 448).to(FP8)
            c = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
            fn = lambda: flag_gems.cutlass_scaled_mm(c, aq, wq.t(), sa.view(-1), sw)  # noqa: E731
        flops, info = 2.0 * m * n * k, {"M": m, "N": n, "K": k}
    elif name == "group_quant":
        x = torch.randn(16384, 7168, device=dev, generator=g).bfloat16()

        def fn():
            flag_gems.per_token_group_quant_fp8(x, 128)
            flag_gems.act_quant_triton(x, 128)

        flops, info = 0.0, {"M": 16384, "K": 7168, "bytes_per_kernel": 16384 * 7168 * (2 + 1 + 4 / 128)}
    elif name == "moe_glue":
        # the two data-movement kernels of the layer at a quarter of the step: 2048 tokens, top-8
        from flaggems_b200.fused.fused_moe import _group_quant_once_then_gather
        from flaggems_b200.fused.moe_sum import moe_sum

        t = 2048
        hid = torch.randn(t, HIDDEN, device=dev, generator=g).bfloat16()
        _, ti = make_router(t, EXPERTS, TOPK)
        ids = ti.to(torch.int32).to(dev)
        sorted_ids, expert_ids, post_pad = moe_align_block_size(ids, _TILE_ROWS, EXPERTS)
        rows = sorted_ids.numel() // _TILE_ROWS * _TILE_ROWS
        routed = torch.randn(t, TOPK, HIDDEN, device=dev, generator=g).bfloat16()
        out = torch.empty(t, HIDDEN, dtype=torch.bfloat16, device=dev)

        def fn():
            _group_quant_once_then_gather(hid, 128, sorted_ids, TOPK, t * TOPK, post_pad, rows)
            moe_sum(routed, out)

        flops, info = 0.0, {"tokens": t, "rows_padded": int(post_pad),
                            "gather_bytes": 2 * int(post_pad) * (HIDDEN + 4 * HIDDEN // 128),
                            "moe_sum_bytes": t * HIDDEN * 2 * (TOPK + 1)}
    else:
        raise SystemExit(f"unknown --workload {name!r}")
    for _ in range(2):
        fn()
    ms = time_events(fn, n_launch)
    line = {"capture_case": name, "launches_timed": n_launch, "ms_per_call": round(ms, 4), **info,
            "device_status": _cabi.device_status()}
    if flops:
        line["tflops"] = round(flops / ms / 1e9, 1)
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-graph", action="store_true", help="issue every step eagerly instead of replaying CUDA graphs")
    ap.add_argument("--passes", type=int, default=5, help="how many times the K timed steps are run (median reported)")
    ap.add_argument("--cpu-tokens", type=int, default=16, help="tokens of the final output compared with the oracle")
    ap.add_argument("--cpu-experts", type=int, default=4,
                    help="experts (with all their routed rows) in the bounded CPU sample at N=1")
    ap.add_argument("--clock-interval-ms", type=int, default=50,
                    help="NVML sampling interval for the clocks record (one sampler thread per rank)")
    ap.add_argument("--no-extras", action="store_true", help="skip the dense GEMM / quant figures at N=1")
    ap.add_argument("--a2a-dispatch", action="store_true",
                    help="send packed rows by NCCL all-to-all instead of storing them to peers from the pack kernel")
    ap.add_argument("--a2a-combine", action="store_true",
                    help="return expert outputs by NCCL all-to-all instead of the fused peer-memory combine")
    ap.add_argument("--workload", default="moe_layer",
                    help="moe_layer (the benchmark) or a single-kernel capture case: moe_gemm1, moe_gemm2, block_mm, "
                         "scaled_mm, group_quant, moe_glue, moe_gemm1_bf16")
    args = ap.parse_args()
    if args.workload != "moe_layer":
        run_capture_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
