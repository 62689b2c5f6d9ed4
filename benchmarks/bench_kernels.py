"""Per-kernel micro-benchmarks with CUDA events: achieved TFLOP/s or GB/s and the fraction of the
measured peaks (MEASURED_PEAKS.json beside the package, or the stated fallback).

    python benchmarks/bench_kernels.py [--only gemm|attn|elementwise|cce|optim] [--iters N] [--json out.json]

Inputs are larger than the 126 MB L2 or the L2 is flushed between iterations (a 256 MB write).
Each number is the mean over ``iters`` launches after 3 warm-up launches, timed on the launching
stream with a synchronize on both sides.  ``--one <name>`` runs a single named case a few times
without timing (the form used under ncu).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from chronicals_b200 import ops  # noqa: E402
from chronicals_b200.config.config import measured_peaks  # noqa: E402
from chronicals_b200.ops import _ext  # noqa: E402

DEV = "cuda"
_FLUSH = None


def flush_l2():
    global _FLUSH
    if _FLUSH is None:
        _FLUSH = torch.empty(256 * 2**20, dtype=torch.uint8, device=DEV)
    _FLUSH.zero_()


def timed(fn, iters=10, flush=True):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    tot = 0.0
    for _ in range(iters):
        if flush:
            flush_l2()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        tot += a.elapsed_time(b)
    return tot / iters


def graph_timed(fn, iters=10):
    """Mean device time of ``fn`` replayed from a CUDA graph (L2 flushed between replays)."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, capture_error_mode="thread_local"):      # the autograd engine runs on its own thread
        fn()
    tot = 0.0
    for _ in range(iters):
        flush_l2()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize()
        tot += a.elapsed_time(b)
    del g
    return tot / iters


def bf(*shape, scale=1.0):
    return (torch.randn(*shape, device=DEV) * scale).to(torch.bfloat16)


GEMM_CASES = {
    # name: (M, N, K, a_mn, b_mn)  -- shapes of the 0.5B / 7B training step, T = 8192 tokens
    "qkv_fwd_0.5b": (8192, 1152, 896, 0, 0), "o_fwd_0.5b": (8192, 896, 896, 0, 0),
    "gateup_fwd_0.5b": (8192, 9728, 896, 0, 0), "down_fwd_0.5b": (8192, 896, 4864, 0, 0),
    "gateup_dgrad_0.5b": (8192, 896, 9728, 0, 1), "down_dgrad_0.5b": (8192, 4864, 896, 0, 1),
    "gateup_wgrad_0.5b": (9728, 896, 8192, 1, 1), "down_wgrad_0.5b": (896, 4864, 8192, 1, 1),
    "qkv_dgrad_0.5b": (8192, 896, 1152, 0, 1), "o_dgrad_0.5b": (8192, 896, 896, 0, 1),
    "gateup_fwd_7b": (8192, 37888, 3584, 0, 0), "down_fwd_7b": (8192, 3584, 18944, 0, 0),
    "square_8k": (8192, 8192, 8192, 0, 0),
}


def gemm_inputs(M, N, K, a_mn, b_mn):
    a = bf(K, M) if a_mn else bf(M, K)
    b = bf(K, N) if b_mn else bf(N, K)
    return a, b


def run_gemm(results, peaks, iters, only=None):
    for name, (M, N, K, a_mn, b_mn) in GEMM_CASES.items():
        if only and only != name:
            continue
        a, b = gemm_inputs(M, N, K, a_mn, b_mn)
        out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
        ms = timed(lambda: ops.gemm(a, b, a_mn=bool(a_mn), b_mn=bool(b_mn), out=out), iters)
        A = a.t() if a_mn else a
        B = b if b_mn else b.t()
        ms_lib = timed(lambda: torch.matmul(A, B, out=out), iters)
        # the CTA-pair kernel alone, with tiles cut along K (stream-K) and restricted to whole tiles
        ms_sk = timed(lambda: ops.gemm(a, b, a_mn=bool(a_mn), b_mn=bool(b_mn), out=out, pair_flags=2), iters)
        ms_whole = timed(lambda: ops.gemm(a, b, a_mn=bool(a_mn), b_mn=bool(b_mn), out=out, pair_flags=1), iters)
        fl = 2.0 * M * N * K
        results.append({"kernel": "gemm_tcgen05", "case": name, "shape": [M, N, K], "ms": ms,
                        "tflops": fl / ms / 1e9, "frac_of_measured_bf16": fl / ms / 1e9 / peaks["bf16_tflops"],
                        "cublas_ms": ms_lib, "cublas_tflops": fl / ms_lib / 1e9, "vs_cublas": ms_lib / ms,
                        "pair_stream_k_ms": ms_sk, "pair_whole_tiles_ms": ms_whole})
        _ext.check_status()


def run_gemm_fp8(results, peaks, iters, only=None):
    """e4m3 GEMM on the tensor cores (pre-quantised operands) against the bf16 GEMM of the same shape."""
    from chronicals_b200.utils.fp8_utils import fp8_rowwise_matmul, rowwise_quantize_e4m3
    for name in ("gateup_fwd_0.5b", "down_fwd_0.5b", "gateup_fwd_7b", "down_fwd_7b", "square_8k"):
        if only and only != name:
            continue
        M, N, K, _, _ = GEMM_CASES[name]
        a, b = bf(M, K), bf(N, K)
        aq, asc = rowwise_quantize_e4m3(a)
        bq, bsc = rowwise_quantize_e4m3(b)
        ms = timed(lambda: fp8_rowwise_matmul(aq, asc, bq, bsc), iters)
        ms_q = timed(lambda: rowwise_quantize_e4m3(a), iters)
        out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
        ms_bf16 = timed(lambda: ops.gemm(a, b, out=out), iters)
        fl = 2.0 * M * N * K
        results.append({"kernel": "gemm2sm_fp8", "case": name, "shape": [M, N, K], "ms": ms, "tflops": fl / ms / 1e9,
                        "frac_of_measured_bf16": fl / ms / 1e9 / peaks["bf16_tflops"], "bf16_gemm_ms": ms_bf16,
                        "speedup_vs_bf16": ms_bf16 / ms, "activation_quant_ms": ms_q})
        _ext.check_status()


def run_gemm_mxfp8(results, peaks, iters, only=None):
    """Block-scaled MXFP8 GEMM (``tcgen05.mma.kind::mxf8f6f4.block_scale``, pre-quantised operands with packed
    e8m0 scales) against the bf16 GEMM of the same shape; also the cost of quantising the activation."""
    from chronicals_b200.utils.fp8_utils import PAIR_TILE_ROWS, mxfp8_block_scaled_matmul, mxfp8_quantize_packed
    for name in ("small_2k", "gateup_fwd_0.5b", "down_fwd_0.5b", "gateup_fwd_7b", "down_fwd_7b", "square_8k"):
        if only and only != name:
            continue
        M, N, K = (2048, 2048, 2048) if name == "small_2k" else GEMM_CASES[name][:3]
        a, b = bf(M, K), bf(N, K)
        aq, sa = mxfp8_quantize_packed(a)
        bq, sb = mxfp8_quantize_packed(b)
        ms1 = timed(lambda: mxfp8_block_scaled_matmul(aq, sa, bq, sb), iters)
        bq, sb = mxfp8_quantize_packed(b, tile_rows=PAIR_TILE_ROWS)
        ms = timed(lambda: mxfp8_block_scaled_matmul(aq, sa, bq, sb, b_tile_rows=PAIR_TILE_ROWS), iters)
        ms_q = timed(lambda: mxfp8_quantize_packed(a), iters)
        out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
        ms_bf16 = timed(lambda: ops.gemm(a, b, out=out), iters)
        fl = 2.0 * M * N * K
        results.append({"kernel": "mxgemm2sm_block_scaled", "case": name, "shape": [M, N, K], "ms": ms, "tflops": fl / ms / 1e9,
                        "frac_of_measured_bf16": fl / ms / 1e9 / peaks["bf16_tflops"], "single_cta_kernel_ms": ms1,
                        "bf16_gemm_ms": ms_bf16,
                        "speedup_vs_bf16": ms_bf16 / ms, "activation_quant_ms": ms_q})
        _ext.check_status()


def run_attn(results, peaks, iters, only=None):
    from chronicals_b200.kernels.flash_attention_optimizer import attention_flops
    cases = {"0.5b_8x1024": (14, 2, 64, [1024] * 8), "0.5b_2x4096": (14, 2, 64, [4096] * 2),
             "7b_2x4096": (28, 4, 128, [4096] * 2), "lora_varlen": (14, 2, 64, None)}
    for name, (hq, hk, d, lens) in cases.items():
        if only and only != name:
            continue
        if lens is None:
            g = torch.Generator().manual_seed(0)
            raw = torch.empty(64).log_normal_(5.5, 1.0, generator=g).clamp(32, 2048).round().long().tolist()
            lens, tot = [], 0
            for l in raw:
                if tot + l > 8192:
                    break
                lens.append(l)
                tot += l
        T = sum(lens)
        qkv = bf(T, (hq + 2 * hk) * d).requires_grad_()
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=DEV)
        g = bf(T, hq * d)
        ms_f = timed(lambda: ops.attention_qkv_packed(qkv.detach(), cu, hq, hk, d), iters)

        def fb():
            o = ops.attention_qkv_packed(qkv, cu, hq, hk, d)
            o.backward(g)
            qkv.grad = None
        ms_fb = timed(fb, iters)
        ff, fbw = attention_flops(lens, hq, d), attention_flops(lens, hq, d, backward=True)
        # the same calls replayed from a CUDA graph, as they run inside the captured training step: eager launches
        # of the short cases are bound by the host (allocation + four to six launches per call)
        ms_f_graph = graph_timed(lambda: ops.attention_qkv_packed(qkv.detach(), cu, hq, hk, d), iters)
        ms_fb_graph = graph_timed(fb, iters)
        rf = {"kernel": "attn_fwd", "case": name, "ms": ms_f, "graph_ms": ms_f_graph, "tflops": ff / ms_f_graph / 1e9,
              "frac_of_measured_bf16": ff / ms_f_graph / 1e9 / peaks["bf16_tflops"]}
        rb = {"kernel": "attn_fwd+bwd", "case": name, "ms": ms_fb, "graph_ms": ms_fb_graph, "tflops": fbw / ms_fb_graph / 1e9,
              "frac_of_measured_bf16": fbw / ms_fb_graph / 1e9 / peaks["bf16_tflops"]}
        if len(set(lens)) == 1:
            # torch's SDPA (its flash / cuDNN back end) on the same box, same run: forward, and forward + backward
            n, L = len(lens), lens[0]
            q = bf(n, hq, L, d).requires_grad_()
            k, v = bf(n, hk, L, d).requires_grad_(), bf(n, hk, L, d).requires_grad_()

            def lib():
                o = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
                o.backward(torch.ones_like(o))

            def lib_fwd():
                with torch.no_grad():
                    torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
            rf["sdpa_fwd_ms"] = timed(lib_fwd, iters)
            rb["sdpa_fwd_bwd_ms"] = timed(lib, iters)
            try:
                rf["sdpa_graph_ms"] = graph_timed(lib_fwd, iters)
                rb["sdpa_graph_ms"] = graph_timed(lib, iters)
                rf["sdpa_over_ours_graph"] = rf["sdpa_graph_ms"] / ms_f_graph
                rb["sdpa_over_ours_graph"] = rb["sdpa_graph_ms"] / ms_fb_graph
            except Exception as e:                           # a back end that cannot be captured
                rf["sdpa_graph_ms"] = rb["sdpa_graph_ms"] = f"not captured: {type(e).__name__}"
        results.append(rf)
        results.append(rb)
        _ext.check_status()


def run_glu(results, peaks, iters, only=None):
    """Gate | up projection + SwiGLU: one GEMM with the activation in its epilogue against GEMM + activation kernel."""
    for name, (M, K, I) in {"mlp_0.5b": (8192, 896, 4864), "mlp_7b": (8192, 3584, 18944)}.items():
        if only and only != name:
            continue
        x, w = bf(M, K), bf(2 * I, K)
        ms_fused = timed(lambda: ops.linear_swiglu(x, w), iters)
        gu = torch.empty(M, 2 * I, dtype=torch.bfloat16, device=DEV)
        ms_gemm = timed(lambda: ops.gemm(x, w, out=gu), iters)
        ms_two = timed(lambda: ops.swiglu(ops.gemm(x, w, out=gu)), iters)
        fl = 2.0 * M * 2 * I * K
        results.append({"kernel": "gateup_gemm+swiglu_epilogue", "case": name, "ms": ms_fused, "tflops": fl / ms_fused / 1e9,
                        "frac_of_measured_bf16": fl / ms_fused / 1e9 / peaks["bf16_tflops"], "gemm_alone_ms": ms_gemm,
                        "gemm_then_activation_ms": ms_two})
        _ext.check_status()


def run_elementwise(results, peaks, iters, only=None):
    T, H, I = 8192, 896, 4864
    bw = peaks["hbm_gbs"]

    def rec(name, ms, nbytes):
        results.append({"kernel": name, "ms": ms, "gbs": nbytes / ms / 1e6, "frac_of_measured_hbm": nbytes / ms / 1e6 / bw})

    x, w = bf(T * 4, H), bf(H)
    rec("rmsnorm_fwd[32768x896]", timed(lambda: ops.rmsnorm(x, w)), 2 * x.numel() * 2)
    xg = x.clone().requires_grad_()
    wg = w.clone().requires_grad_()
    y = ops.rmsnorm(xg, wg)
    gy = torch.randn_like(y)
    rec("rmsnorm_bwd[32768x896]", timed(lambda: torch.autograd.grad(y, (xg, wg), gy, retain_graph=True)), 3 * x.numel() * 2)
    gu = bf(T, 2 * I)
    rec("swiglu_fwd[8192x4864]", timed(lambda: ops.swiglu(gu)), (gu.numel() + gu.numel() // 2) * 2)
    gug = gu.clone().requires_grad_()
    a = ops.swiglu(gug)
    ga = torch.randn_like(a)
    rec("swiglu_bwd[8192x4864]", timed(lambda: torch.autograd.grad(a, gug, ga, retain_graph=True)), (2 * gu.numel() + a.numel()) * 2)
    from chronicals_b200.ops import ref
    qkv = bf(T * 4, 1152)
    cos, sin = ref.rope_cache(1024, 64, 1e6, device=DEV)
    pos = (torch.arange(T * 4, device=DEV) % 1024)
    rec("qk_rope[32768x(14+2)x64]", timed(lambda: ops.qk_rope_(qkv, cos, sin, pos, 14, 2, 64)), 2 * T * 4 * 1024 * 2)


def run_cce(results, peaks, iters, only=None):
    """Fused linear cross-entropy on the benchmark's head (8192 tokens x 151,936 words), both forms: logits
    resident in bf16 between forward and backward (3 GEMM passes), and never held (4 passes: the backward
    recomputes them in chunks)."""
    T, H, V = 8192, 896, 151936
    h = bf(T, H).requires_grad_()
    w = bf(V, H, scale=0.02).requires_grad_()
    y = torch.randint(0, V, (T,), device=DEV)
    fl = 2.0 * T * H * V
    keep = ops.CCE_RESIDENT_BYTES
    for form, limit, passes in (("logits resident", 1 << 40, 3), ("no logits", 0, 4)):
        ops.CCE_RESIDENT_BYTES = limit
        ms_f = timed(lambda: ops.linear_cross_entropy(h.detach(), w.detach(), y), iters, flush=False)

        def fb():
            ops.linear_cross_entropy(h, w, y).backward()
            h.grad = w.grad = None
        ms_fb = timed(fb, max(3, iters // 2), flush=False)
        results.append({"kernel": "cce_fwd", "case": f"0.5b, {form}", "ms": ms_f, "tflops": fl / ms_f / 1e9,
                        "frac_of_measured_bf16": fl / ms_f / 1e9 / peaks["bf16_tflops"]})
        results.append({"kernel": "cce_fwd+bwd", "case": f"0.5b, {form} ({passes} GEMM passes)", "ms": ms_fb,
                        "tflops": passes * fl / ms_fb / 1e9,
                        "frac_of_measured_bf16": passes * fl / ms_fb / 1e9 / peaks["bf16_tflops"]})
    ops.CCE_RESIDENT_BYTES = keep
    _ext.check_status()


def run_optim(results, peaks, iters, only=None):
    from chronicals_b200.optimizers.fused_adamw import FusedAdamW
    n = 400_000_000
    p = torch.nn.Parameter(torch.zeros(n, device=DEV, dtype=torch.bfloat16))
    p.grad = torch.randn(n, device=DEV).to(torch.bfloat16)
    opt = FusedAdamW([p], lr=1e-4, max_grad_norm=1.0)
    ms = timed(opt.step, iters, flush=False)
    nbytes = n * (2 + 2 + 2 + 4 + 4 + 2 + 4 + 4)         # sq-norm read + p,g,m,v read + p,m,v write
    results.append({"kernel": "adamw_multi + grad clip [400M bf16]", "ms": ms, "gbs": nbytes / ms / 1e6,
                    "frac_of_measured_hbm": nbytes / ms / 1e6 / peaks["hbm_gbs"]})
    torch_p = torch.nn.Parameter(torch.zeros(n, device=DEV, dtype=torch.bfloat16))
    torch_p.grad = p.grad
    o2 = torch.optim.AdamW([torch_p], lr=1e-4, fused=True)
    results[-1]["torch_fused_adamw_ms"] = timed(o2.step, iters, flush=False)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default=None)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--json", default=None)
    ap.add_argument("--one", default=None, help="run one GEMM case 3 times without timing (for ncu); mx:<case> runs the block-scaled MXFP8 GEMM")
    args = ap.parse_args()
    peaks = measured_peaks()
    if args.one and args.one.startswith("attn"):
        hq, hk, d, L, n = 14, 2, 64, 1024, 8
        T = n * L
        qkv = bf(T, (hq + 2 * hk) * d).requires_grad_()
        cu = torch.arange(0, T + 1, L, dtype=torch.int32, device=DEV)
        g = bf(T, hq * d)
        for _ in range(2):
            o = ops.attention_qkv_packed(qkv, cu, hq, hk, d)
            o.backward(g)
            qkv.grad = None
        torch.cuda.synchronize()
        _ext.check_status()
        print("ok")
        return
    if args.one and args.one.startswith("glu:"):                  # glu:mlp_0.5b - the GEMM with the SwiGLU epilogue
        M, K, I = {"mlp_0.5b": (8192, 896, 4864), "mlp_7b": (8192, 3584, 18944)}[args.one.split(":", 1)[1]]
        x, w = bf(M, K), bf(2 * I, K)
        for _ in range(3):
            ops.linear_swiglu(x, w)
        torch.cuda.synchronize()
        _ext.check_status()
        print("ok")
        return
    if args.one and args.one.startswith(("mx:", "mxp:")):
        from chronicals_b200.utils.fp8_utils import PAIR_TILE_ROWS, mxfp8_block_scaled_matmul, mxfp8_quantize_packed
        tile = PAIR_TILE_ROWS if args.one.startswith("mxp:") else 128          # mxp: the CTA-pair kernel
        M, N, K = GEMM_CASES[args.one.split(":", 1)[1]][:3]
        aq, sa = mxfp8_quantize_packed(bf(M, K))
        bq, sb = mxfp8_quantize_packed(bf(N, K), tile_rows=tile)
        for _ in range(3):
            mxfp8_block_scaled_matmul(aq, sa, bq, sb, b_tile_rows=tile)
        torch.cuda.synchronize()
        _ext.check_status()
        print("ok")
        return
    if args.one and args.one.startswith("fp8:"):
        from chronicals_b200.utils.fp8_utils import fp8_rowwise_matmul, rowwise_quantize_e4m3
        M, N, K = GEMM_CASES[args.one.split(":", 1)[1]][:3]
        aq, asc = rowwise_quantize_e4m3(bf(M, K))
        bq, bsc = rowwise_quantize_e4m3(bf(N, K))
        for _ in range(3):
            fp8_rowwise_matmul(aq, asc, bq, bsc)
        torch.cuda.synchronize()
        _ext.check_status()
        print("ok")
        return
    if args.one:
        # "<case>": the dispatcher's choice; "single:<case>": the single-CTA kernel; "pair:<case>": CTA pairs, whole
        # tiles; "split:<case>": CTA pairs with the last round cut along K
        mode, _, case = args.one.rpartition(":")
        M, N, K, a_mn, b_mn = GEMM_CASES[case]
        a, b = gemm_inputs(M, N, K, a_mn, b_mn)
        out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
        kw = {"single": {"block_n": 256}, "pair": {"pair_flags": 1}, "split": {"pair_flags": 2}}.get(mode, {})
        for _ in range(3):
            ops.gemm(a, b, a_mn=bool(a_mn), b_mn=bool(b_mn), out=out, **kw)
        torch.cuda.synchronize()
        _ext.check_status()
        print("ok")
        return
    class _Live(list):
        def append(self, r):
            super().append(r)
            extra = "".join(f"  {k}={v:.3f}" if isinstance(v, float) else f"  {k}={v}" for k, v in r.items()
                            if k not in ("kernel", "case", "ms"))
            print(f"{r['kernel']:<28s} {r.get('case', ''):<22s} {r['ms']:8.3f} ms{extra}", flush=True)

    print(f"peaks ({peaks['source']}): bf16 {peaks['bf16_tflops']} TFLOP/s, HBM {peaks['hbm_gbs']} GB/s", flush=True)
    results = _Live()
    groups = {"gemm": run_gemm, "gemm_fp8": run_gemm_fp8, "gemm_mxfp8": run_gemm_mxfp8, "attn": run_attn, "glu": run_glu, "elementwise": run_elementwise, "cce": run_cce, "optim": run_optim}
    for name, fn in groups.items():
        if args.only and args.only != name:
            continue
        fn(results, peaks, args.iters)
    if args.json:
        with open(args.json, "w") as f:
            json.dump({"peaks": peaks, "results": list(results)}, f, indent=1)


if __name__ == "__main__":
    main()
