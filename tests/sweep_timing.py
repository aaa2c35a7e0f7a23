"""Timing sweep over the benchmark configurations (CUDA events, CUDA-graph replays, no profiler).

    python tests/sweep_timing.py gemv [--ref]     decode GEMV, all block types
    python tests/sweep_timing.py gemm [--ref]     tensor-core GEMM (ggml_mul_mat_a8 / dequantize-matmul route)
    python tests/sweep_timing.py moe  [--ref]     OLMoE-shaped ggml_moe_a8 (gate/up and down GEMMs)
    python tests/sweep_timing.py dequant [--ref]  standalone ggml_dequantize (all types) and the q8_1 quantizer

One JSON line per case.  Every case rotates over enough seeded weight copies that a launch reads
its weights cold (> 300 MB per graph); "us" is the mean per call.  With --ref the reference
plugin's own CUDA kernels (oracle/_ref/_C_gguf_ref.so, built by oracle/build_ref.py where the
reference sources are present) are timed the same way next to ours.  This file lives under
tests/ because it may load that checker library; nothing in the package does.
"""
from __future__ import annotations

import json
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT / "vllm-gguf-plugin-prism_b200"))
sys.path.insert(0, str(ROOT))

from gguf_b200 import capi, synth  # noqa: E402

DEV = "cuda"
Q4_0, Q8_0, Q4_K, Q6_K, IQ2_XXS, IQ4_XS = 2, 8, 12, 14, 16, 23

GEMV_CASES = [(Q4_K, 57344, 4096, 1), (Q8_0, 3072, 1024, 1), (Q4_K, 14336, 4096, 1), (Q4_K, 4096, 14336, 1),
              (Q6_K, 37888, 3584, 1), (Q6_K, 3584, 18944, 1), (IQ4_XS, 37888, 3584, 1), (IQ4_XS, 3584, 18944, 1),
              (IQ2_XXS, 28672, 8192, 1), (IQ2_XXS, 8192, 28672, 1), (Q4_0, 2048, 2048, 1), (Q4_0, 16384, 4096, 1),
              (Q4_K, 14336, 4096, 2), (Q4_K, 14336, 4096, 4), (Q4_K, 14336, 4096, 8)]
GEMM_CASES = [("mmq", Q4_K, 14336, 4096, 2048), ("mmq", Q4_K, 14336, 4096, 512), ("mmq", Q4_K, 4096, 14336, 512),
              ("mmq", Q4_K, 14336, 4096, 64), ("mmq", Q4_K, 4096, 14336, 64), ("mmq", Q4_K, 14336, 4096, 8), ("mmq", Q4_K, 4096, 14336, 8),
              ("mmq", Q4_K, 14336, 4096, 4), ("mmq", Q4_K, 14336, 4096, 16),
              ("mmq", Q6_K, 37888, 3584, 256), ("mmq", Q8_0, 14336, 4096, 512), ("mmq", Q4_0, 14336, 4096, 512),
              ("dqmm", IQ2_XXS, 28672, 8192, 128), ("dqmm", IQ2_XXS, 8192, 28672, 128), ("dqmm", IQ4_XS, 37888, 3584, 256)]


def peaks():
    f = ROOT / "MEASURED_PEAKS.json"
    p = json.loads(f.read_text()) if f.exists() else {}
    return float(p.get("hbm_gbs", 6650.0)), float(p.get("bf16_tflops", 1590.0))


def graph_time(calls, reps=None):
    """Mean seconds per call of a list of zero-argument callables, replayed as one CUDA graph
    (run eagerly if the calls cannot be captured)."""
    s = torch.cuda.Stream()
    reps = reps or 10
    with torch.cuda.stream(s):
        for c in calls[:2]:
            c()
        s.synchronize()

        def eager():
            for c in calls:
                c()

        run = eager
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=s):
                eager()
            run = g.replay
        except Exception:
            torch.cuda.synchronize()
        for _ in range(3):
            run()
        s.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(s)
        for _ in range(reps):
            run()
        e1.record(s)
        s.synchronize()
    return e0.elapsed_time(e1) / 1e3 / (reps * len(calls))


def copies(t, n, k, budget=300e6):
    base = synth.make_weight(t, n, k, seed=1)
    ncopy = max(2, int(budget // base.nbytes) + 1)
    return base.nbytes, [torch.from_numpy(base).to(DEV).roll(c, 0).contiguous() for c in range(ncopy)]


def load_ref():
    so = ROOT / "oracle" / "_ref" / "_C_gguf_ref.so"
    if not so.exists():
        raise SystemExit("--ref needs oracle/_ref/_C_gguf_ref.so (python oracle/build_ref.py)")
    torch.ops.load_library(str(so))
    return torch.ops._C_gguf_ref


def sweep_gemv(ref):
    hbm, _ = peaks()
    for (t, n, k, m) in GEMV_CASES:
        wb, ws = copies(t, n, k, 600e6)
        x = torch.from_numpy(synth.make_activation(m, k, seed=0)).to(DEV)
        prep = capi.gemv_prepare(x, t)
        y = torch.empty((m, n), dtype=torch.float16, device=DEV)
        tk = graph_time([lambda w=w: capi.gemv_prepared(w, prep, t, m, n, k, out=y) for w in ws])
        tc = graph_time([lambda w=w: capi.mul_mat_vec_a8(w, x, t, n) for w in ws])
        r = dict(op="gemv", type=synth.NAMES[t], N=n, K=k, M=m, MB=wb / 1e6, us_kernel=tk * 1e6, GBs_kernel=wb / tk / 1e9,
                 frac_of_measured_hbm=wb / tk / 1e9 / hbm, us_call=tc * 1e6, GBs_call=wb / tc / 1e9, status=capi.last_status())
        if ref is not None:
            tr = graph_time([lambda w=w: ref.ggml_mul_mat_vec_a8(w, x, t, n) for w in ws])
            r.update(us_reference=tr * 1e6, speedup_call=tr / tc)
        print(json.dumps(r), flush=True)
        del ws
        torch.cuda.empty_cache()


def sweep_gemm(ref):
    _, tf = peaks()
    for (op, t, n, k, m) in GEMM_CASES:
        wb, ws = copies(t, n, k)
        x = torch.from_numpy(synth.make_activation(m, k, seed=0)).to(DEV)
        fn = capi.mul_mat_a8 if op == "mmq" else capi.dequant_matmul
        tm = graph_time([lambda w=w: fn(w, x, t, n) for w in ws])
        flops = 2.0 * m * n * k
        r = dict(op=op, type=synth.NAMES[t], N=n, K=k, M=m, us=tm * 1e6, tflops=flops / tm / 1e12,
                 frac_of_measured_16bit_peak=flops / tm / 1e12 / tf, weight_GBs=wb / tm / 1e9, status=capi.last_status())
        if ref is not None:
            if op == "mmq":
                tr = graph_time([lambda w=w: ref.ggml_mul_mat_a8(w, x, t, n) for w in ws[:4]], reps=3)
            else:
                tr = graph_time([lambda w=w: x @ ref.ggml_dequantize(w, t, n, k, torch.float16).T for w in ws[:4]], reps=3)
            r.update(us_reference=tr * 1e6, speedup=tr / tm)
        print(json.dumps(r), flush=True)
        del ws
        torch.cuda.empty_cache()


def sweep_moe(ref):
    e_cnt, top_k, hid, inter, tokens = 64, 8, 2048, 1024, 256   # OLMoE-1B-7B shape, 256 tokens
    t = Q4_0
    w13 = torch.from_numpy(np.stack([synth.make_weight(t, 2 * inter, hid, seed=100 + e) for e in range(e_cnt)])).to(DEV)
    w2 = torch.from_numpy(np.stack([synth.make_weight(t, hid, inter, seed=200 + e) for e in range(e_cnt)])).to(DEV)
    x1 = torch.from_numpy(synth.make_activation(tokens, hid, seed=1)).to(DEV)
    x2 = torch.from_numpy(synth.make_activation(tokens * top_k, inter, seed=2)).to(DEV)
    _, ids = synth.make_routing(tokens, e_cnt, top_k, 0)
    blk = capi.lib().gguf_b200_moe_block_size(t)
    s, e, n = [torch.from_numpy(a).to(DEV) for a in synth.moe_align_block_size(ids, blk, e_cnt)]
    t1 = graph_time([lambda: capi.moe_a8(x1, w13, s, e, n, t, 2 * inter, top_k, tokens)] * 4)
    t2 = graph_time([lambda: capi.moe_a8(x2, w2, s, e, n, t, hid, 1, tokens * top_k)] * 4)
    r = dict(op="moe_a8 Q4_0 64 experts top-8, 256 tokens", us_gate_up=t1 * 1e6, us_down=t2 * 1e6,
             weight_GBs_gate_up=w13.numel() / t1 / 1e9, weight_GBs_down=w2.numel() / t2 / 1e9, status=capi.last_status())
    if ref is not None:
        s4, e4, n4 = [torch.from_numpy(a).to(DEV) for a in synth.moe_align_block_size(ids, 4, e_cnt)]
        r1 = graph_time([lambda: ref.ggml_moe_a8(x1, w13, s4, e4, n4, t, 2 * inter, top_k, tokens)] * 2, reps=3)
        r2 = graph_time([lambda: ref.ggml_moe_a8(x2, w2, s4, e4, n4, t, hid, 1, tokens * top_k)] * 2, reps=3)
        r.update(us_reference_gate_up=r1 * 1e6, us_reference_down=r2 * 1e6)
    print(json.dumps(r), flush=True)
    # decode: a few tokens, every (token, expert) pair is one GEMV (ggml_moe_a8_vec)
    for tk in (1, 4, 16):
        xs = x1[:tk].contiguous()
        tid = torch.from_numpy(np.ascontiguousarray(ids[:tk])).to(DEV).to(torch.int32)
        tv = graph_time([lambda: capi.moe_a8_vec(xs, w13, tid, top_k, t, 2 * inter, tk)] * 4)
        rv = dict(op="moe_a8_vec Q4_0 gate/up", tokens=tk, us=tv * 1e6,
                  weight_GBs=tk * top_k * 2 * inter * (hid // 32 * 18) / tv / 1e9, status=capi.last_status())
        if ref is not None:
            rr = graph_time([lambda: ref.ggml_moe_a8_vec(xs, w13, tid, top_k, t, 2 * inter, tk)] * 2, reps=3)
            rv.update(us_reference=rr * 1e6)
        print(json.dumps(rv), flush=True)


def sweep_dequant(ref):
    hbm, _ = peaks()
    for (t, n, k) in [(Q4_K, 14336, 4096), (Q4_0, 14336, 4096), (Q8_0, 14336, 4096), (Q6_K, 37888, 3584),
                      (IQ4_XS, 37888, 3584), (IQ2_XXS, 28672, 8192)]:
        wb, ws = copies(t, n, k, 200e6)
        ws = ws[:4]
        td = graph_time([lambda w=w: capi.dequantize(w, t, n, k, torch.float16) for w in ws])
        moved = wb + n * k * 2      # packed weights in, fp16 values out
        r = dict(op="dequantize->f16", type=synth.NAMES[t], N=n, K=k, us=td * 1e6, GBs=moved / td / 1e9,
                 frac_of_measured_hbm=moved / td / 1e9 / hbm)
        if ref is not None:
            tr = graph_time([lambda w=w: ref.ggml_dequantize(w, t, n, k, torch.float16) for w in ws], reps=5)
            r.update(us_reference=tr * 1e6, speedup=tr / td)
        print(json.dumps(r), flush=True)
        del ws
        torch.cuda.empty_cache()
    for (m, k) in [(1, 4096), (512, 4096), (2048, 4096)]:
        x = torch.from_numpy(synth.make_activation(m, k, seed=0)).to(DEV)
        tq = graph_time([lambda: capi.quantize_q8_1(x)] * 8)
        moved = m * k * 2 + m * k // 32 * 36
        print(json.dumps(dict(op="quantize_q8_1 (36-byte blocks)", M=m, K=k, us=tq * 1e6, GBs=moved / tq / 1e9)), flush=True)


def main():
    what = sys.argv[1] if len(sys.argv) > 1 else "gemm"
    ref = load_ref() if "--ref" in sys.argv else None
    {"gemv": sweep_gemv, "gemm": sweep_gemm, "moe": sweep_moe, "dequant": sweep_dequant}[what](ref)


if __name__ == "__main__":
    main()
