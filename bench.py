"""Benchmark of the GGUF quantized-matmul hot path on B200.

    python bench.py --gpus N --steps K --warmup W            (this library)
    python bench.py --impl reference --gpus N --steps K ...  (the reference's CPU route)
    python bench.py --sweep gemv|gemm|moe|dequant [--ref]    (timing sweeps over all configurations)
    python bench.py --ncu-case op,type,N,K,M                 (six plain calls: a small target for ncu)

Workload (headline): decode GEMV on Q4_K weights with the Llama-3-8B linear shapes
(K=4096 -> N=14336 and K=14336 -> N=4096, one fp16 activation vector, seeded synthetic
blocks).  One "step" is one pass over 16 independently generated copies of each of the two
matrices (32 GEMV calls, 1.06 GB of packed weights), so every call reads weights that have
been evicted from the 126 MB L2 since their last use.  A step is captured once in a CUDA
graph and replayed, as a serving engine does for decode.

Metric: quantized-weight bytes per second (GB/s), the numerator the GEMV roofline uses.
  value     inputs resident in HBM, whole step (activation quantization + GEMV kernels)
  e2e       the same step through the public API with HOST activations: pinned host -> device
            copy of the step's activations and device -> host read of its outputs inside the
            timed region
  roofline  the GEMV kernel alone (activations pre-quantized), algorithmic bytes / duration,
            against the measured copy bandwidth of MEASURED_PEAKS.json
  cpu_baseline  the reference's CPU route (gguf-py dequantize + torch fp32 matmul) on the
            host cores, on a bounded sample of the same workload

N > 1: the same matrices column-sharded over the ranks (rank r holds rows [r*N/g, (r+1)*N/g),
the reference's tensor-parallel slicing rule, quantization/params.py:227-236); total work is
fixed ("strong").  The all-gather of the output slices is part of the GEMV kernel (tagged
packets stored into every rank's memory over NVLink), and the 32 calls of a step form ONE
dependent chain, as in a decoder: up_c reads seed + s * gathered(down_{c-1}), down_c reads
seed + s * gathered(up_c), so every call consumes the whole vector gathered by the call before
it.  All seeds change sign every step (one tiny kernel inside the step), so a packet left over
from the previous step could not pass for a fresh one.  After the timed regions every rank
checks gathered vectors, on rows taken from every rank's slice, against the CPU oracle.

`extras` carries, at every N, the largest configuration (IQ2_XXS 28672x8192 / 8192x28672,
column-sharded): tokens/s = M / (t_up + t_down) for M = 1 and M = 128 with the gathers inside
the time; at N = 1 also tensor-core GEMM and MoE figures and the reference's own CUDA kernels
timed on the same inputs.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for _p in (str(ROOT), str(ROOT / "vllm-gguf-plugin-prism_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import numpy as np  # noqa: E402

Q4_0, Q8_0, Q4_K, Q6_K, IQ2_XXS, IQ4_XS = 2, 8, 12, 14, 16, 23
SHAPES = [(14336, 4096), (4096, 14336)]  # (N rows, K) of the two Llama-3-8B linear shapes
COPIES = 16
METRIC = "quant GEMV HBM GB/s (quantized-weight bytes / s), Q4_K decode, Llama-3-8B linear shapes"
CHAIN_SCALE = 2.0 ** -12   # weight of the gathered vector in the next call's activations (N > 1)


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    d = json.loads(p.read_text()) if p.exists() else {}
    which = "measured" if d else "fallback"
    return float(d.get("hbm_gbs", 6650.0)), float(d.get("bf16_tflops", 1590.0)), which


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 50 ms while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc, self.t_mark = index, [], None, None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
            time.sleep(1.2)   # the sampler is running before the timed region starts
        except Exception:
            self.proc = None
        return self

    def mark(self):
        """Samples from here on count as 'under load'."""
        self.t_mark = len(self.rows)

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self):
        rows = self.rows[self.t_mark:] if self.t_mark is not None else self.rows
        sm = [float(r[0]) for r in rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for r in rows if len(r) >= 6 for i in range(4) if r[2 + i].lower().startswith("active")})
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


# --------------------------------------------------------------------------------------------
# the reference's CPU route (reference arm and cpu_baseline)
# --------------------------------------------------------------------------------------------

def cpu_route_sample(n_rows: int, k: int, threads: int):
    """gguf-py dequantize + torch fp32 matmul (the reference's CPU route) on one Q4_K matrix."""
    import torch

    from gguf_b200 import synth
    from oracle import cpu

    torch.set_num_threads(threads)
    w = synth.make_weight(Q4_K, n_rows, k, seed=0)
    x = torch.from_numpy(synth.make_activation(1, k, seed=0)).float()
    t0 = time.perf_counter()
    wd = cpu.gguf_py_dequantize(w, Q4_K)
    t1 = time.perf_counter()
    y = x @ torch.from_numpy(wd).T
    t2 = time.perf_counter()
    return w.nbytes, t1 - t0, t2 - t1, float(y.abs().sum())


def run_reference_arm(args):
    """The reference's own CPU implementation of the path, timed on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    n_rows, k = SHAPES[0]
    rows = max(n_rows // 4, 256)  # bounded sample: a quarter of one matrix per step
    for _ in range(max(args.warmup, 1)):
        cpu_route_sample(256, k, threads)
    tot_b, tot_t = 0, 0.0
    for _ in range(args.steps):
        b, td, tm, _ = cpu_route_sample(rows, k, threads)
        tot_b += b
        tot_t += td + tm
    val = tot_b / tot_t / 1e9
    sample = f"{rows}x{k} Q4_K rows per step (1/4 of the 14336x4096 matrix), gguf-py dequantize + torch fp32 matmul"
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": tot_t / args.steps * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "Q4_K GEMV M=1, Llama-3-8B shapes", "path": "reference CPU route"},
            "cpu_baseline": {"value": val, "unit": "GB/s", "cores": threads, "kind": "reference", "sample": sample},
            "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------
# timing helpers
# --------------------------------------------------------------------------------------------

def graph_time(calls, reps=10, warm=3):
    """Mean seconds per call of a list of zero-argument callables, replayed as one CUDA graph
    (run eagerly if the calls cannot be captured).  CUDA events on the launching stream."""
    import torch

    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
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
        for _ in range(warm):
            run()
        s.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(s)
        for _ in range(reps):
            run()
        e1.record(s)
        s.synchronize()
    return e0.elapsed_time(e1) / 1e3 / (reps * len(calls))


def rolled_copies(t, n, k, budget=300e6, seed=1, dev="cuda"):
    """Enough row-rotated device copies of one seeded matrix that a pass over them reads > budget bytes."""
    import torch

    from gguf_b200 import synth

    base = synth.make_weight(t, n, k, seed=seed)
    ncopy = max(2, int(budget // base.nbytes) + 1)
    first = torch.from_numpy(base).to(dev)
    return base.nbytes, [first] + [first.roll(c, 0).contiguous() for c in range(1, ncopy)]


def load_ref_cuda():
    """The reference plugin's own CUDA extension, built from its sources by oracle/build_ref.py
    (a baseline to time next to this library; None if the file is absent)."""
    import torch

    so = ROOT / "oracle" / "_ref" / "_C_gguf_ref.so"
    if not so.exists():
        return None
    torch.ops.load_library(str(so))
    return torch.ops._C_gguf_ref


# --------------------------------------------------------------------------------------------
# sweeps (one JSON line per case)
# --------------------------------------------------------------------------------------------

GEMV_CASES = [(Q4_K, 57344, 4096, 1), (Q8_0, 3072, 1024, 1), (Q4_K, 14336, 4096, 1), (Q4_K, 4096, 14336, 1),
              (Q6_K, 37888, 3584, 1), (Q6_K, 3584, 18944, 1), (IQ4_XS, 37888, 3584, 1), (IQ4_XS, 3584, 18944, 1),
              (IQ2_XXS, 28672, 8192, 1), (IQ2_XXS, 8192, 28672, 1), (Q4_0, 2048, 2048, 1), (Q4_0, 16384, 4096, 1),
              (Q4_K, 14336, 4096, 2), (Q4_K, 14336, 4096, 4), (Q4_K, 14336, 4096, 8)]
GEMM_CASES = [("mmq", Q4_K, 14336, 4096, 2048), ("mmq", Q4_K, 14336, 4096, 512), ("mmq", Q4_K, 4096, 14336, 512),
              ("mmq", Q4_K, 14336, 4096, 64), ("mmq", Q4_K, 4096, 14336, 64), ("mmq", Q4_K, 14336, 4096, 8), ("mmq", Q4_K, 4096, 14336, 8),
              ("mmq", Q4_K, 14336, 4096, 4), ("mmq", Q4_K, 14336, 4096, 16),
              ("mmq", Q6_K, 37888, 3584, 256), ("mmq", Q6_K, 3584, 18944, 256), ("mmq", Q8_0, 14336, 4096, 512), ("mmq", Q4_0, 14336, 4096, 512),
              ("dqmm", IQ2_XXS, 28672, 8192, 128), ("dqmm", IQ2_XXS, 8192, 28672, 128), ("dqmm", IQ4_XS, 37888, 3584, 256),
              ("dqmm", IQ4_XS, 3584, 18944, 256), ("mmq", 10, 14336, 4096, 512), ("mmq", 11, 14336, 4096, 512), ("mmq", 13, 14336, 4096, 512),
              ("mmq", 3, 14336, 4096, 512), ("mmq", 6, 14336, 4096, 512), ("mmq", 7, 14336, 4096, 512)]   # 10, 11, 13 = Q2_K, Q3_K, Q5_K; 3, 6, 7 = Q4_1, Q5_0, Q5_1


def sweep_gemv(ref):
    import torch

    from gguf_b200 import capi, synth

    hbm, _, _ = peaks()
    for (t, n, k, m) in GEMV_CASES:
        wb, ws = rolled_copies(t, n, k, 600e6)
        x = torch.from_numpy(synth.make_activation(m, k, seed=0)).to("cuda")
        prep = capi.gemv_prepare(x, t)
        y = torch.empty((m, n), dtype=torch.float16, device="cuda")
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
    import torch

    from gguf_b200 import capi, synth

    _, tf, _ = peaks()
    for (op, t, n, k, m) in GEMM_CASES:
        wb, ws = rolled_copies(t, n, k)
        x = torch.from_numpy(synth.make_activation(m, k, seed=0)).to("cuda")
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


def moe_case(dev="cuda"):
    """The OLMoE-1B-7B MoE configuration: 64 experts, top-8, hidden 2048, intermediate 1024, Q4_0, 256 tokens."""
    import torch

    from gguf_b200 import capi, synth

    e_cnt, top_k, hid, inter, tokens = 64, 8, 2048, 1024, 256
    t = Q4_0
    w13 = torch.from_numpy(np.stack([synth.make_weight(t, 2 * inter, hid, seed=100 + e) for e in range(e_cnt)])).to(dev)
    w2 = torch.from_numpy(np.stack([synth.make_weight(t, hid, inter, seed=200 + e) for e in range(e_cnt)])).to(dev)
    x1 = torch.from_numpy(synth.make_activation(tokens, hid, seed=1)).to(dev)
    x2 = torch.from_numpy(synth.make_activation(tokens * top_k, inter, seed=2)).to(dev)
    tw, ids = synth.make_routing(tokens, e_cnt, top_k, 0)
    blk = capi.lib().gguf_b200_moe_block_size(t)
    ours = [torch.from_numpy(a).to(dev) for a in synth.moe_align_block_size(ids, blk, e_cnt)]
    ref4 = [torch.from_numpy(a).to(dev) for a in synth.moe_align_block_size(ids, 4, e_cnt)]   # the reference's own block size
    return dict(t=t, e_cnt=e_cnt, top_k=top_k, hid=hid, inter=inter, tokens=tokens, w13=w13, w2=w2, x1=x1, x2=x2, ids=ids,
                ours=ours, ref4=ref4, ids_dev=torch.from_numpy(ids).to(dev), tw_dev=torch.from_numpy(tw).to(dev))


def moe_times(c, ref):
    from gguf_b200 import capi

    t, top_k, hid, inter, tokens = c["t"], c["top_k"], c["hid"], c["inter"], c["tokens"]
    s, e, n = c["ours"]
    t1 = graph_time([lambda: capi.moe_a8(c["x1"], c["w13"], s, e, n, t, 2 * inter, top_k, tokens)] * 4)
    t2 = graph_time([lambda: capi.moe_a8(c["x2"], c["w2"], s, e, n, t, hid, 1, tokens * top_k)] * 4)
    hbm, tf, _ = peaks()
    ops1, ops2 = 2.0 * tokens * top_k * 2 * inter * hid, 2.0 * tokens * top_k * hid * inter
    r = dict(op="moe_a8 Q4_0 64 experts top-8, 256 tokens", us_gate_up=t1 * 1e6, us_down=t2 * 1e6,
             weight_GBs_gate_up=c["w13"].numel() / t1 / 1e9, weight_GBs_down=c["w2"].numel() / t2 / 1e9,
             frac_of_measured_hbm_gate_up=c["w13"].numel() / t1 / 1e9 / hbm, frac_of_measured_hbm_down=c["w2"].numel() / t2 / 1e9 / hbm,
             tflops_gate_up=ops1 / t1 / 1e12, tflops_down=ops2 / t2 / 1e12, bound="hbm (32 rows per expert)", status=capi.last_status())
    # the whole step of a layer (alignment, both GEMMs, activation, routing weights, top-k sum) in one call
    tf_ = graph_time([lambda: capi.fused_moe(c["x1"], c["w13"], c["w2"], c["ids_dev"], c["tw_dev"], t, t)] * 4)
    r.update(us_fused_step=tf_ * 1e6, weight_GBs_fused_step=(c["w13"].numel() + c["w2"].numel()) / tf_ / 1e9,
             frac_of_measured_hbm_fused_step=(c["w13"].numel() + c["w2"].numel()) / tf_ / 1e9 / hbm)
    if ref is not None:
        import torch

        s4, e4, n4 = c["ref4"]
        r1 = graph_time([lambda: ref.ggml_moe_a8(c["x1"], c["w13"], s4, e4, n4, t, 2 * inter, top_k, tokens)] * 2, reps=3)
        r2 = graph_time([lambda: ref.ggml_moe_a8(c["x2"], c["w2"], s4, e4, n4, t, hid, 1, tokens * top_k)] * 2, reps=3)
        r.update(us_reference_gate_up=r1 * 1e6, us_reference_down=r2 * 1e6, speedup_gate_up=r1 / t1, speedup_down=r2 / t2)

        def ref_step():   # the reference's sequence with its own kernels (alignment precomputed, activation / weighting / sum in torch)
            o = ref.ggml_moe_a8(c["x1"], c["w13"], s4, e4, n4, t, 2 * inter, top_k, tokens)
            a = (torch.nn.functional.silu(o[:, :inter]) * o[:, inter:]).contiguous()
            o = ref.ggml_moe_a8(a, c["w2"], s4, e4, n4, t, hid, 1, tokens * top_k)
            return (o.view(tokens, top_k, hid) * c["tw_dev"].view(tokens, top_k, 1).to(o.dtype)).sum(1)

        rs = graph_time([ref_step] * 2, reps=3)
        r.update(us_reference_step=rs * 1e6, speedup_step=rs / tf_)
    return r


def sweep_moe(ref):
    import torch

    from gguf_b200 import capi

    c = moe_case()
    print(json.dumps(moe_times(c, ref)), flush=True)
    t, top_k, hid, inter = c["t"], c["top_k"], c["hid"], c["inter"]
    # decode: a few tokens, every (token, expert) pair is one GEMV (ggml_moe_a8_vec)
    for tk in (1, 4, 16):
        xs = c["x1"][:tk].contiguous()
        tid = torch.from_numpy(np.ascontiguousarray(c["ids"][:tk])).to("cuda").to(torch.int32)
        tv = graph_time([lambda: capi.moe_a8_vec(xs, c["w13"], tid, top_k, t, 2 * inter, tk)] * 4)
        rv = dict(op="moe_a8_vec Q4_0 gate/up", tokens=tk, us=tv * 1e6,
                  weight_GBs=tk * top_k * 2 * inter * (hid // 32 * 18) / tv / 1e9, status=capi.last_status())
        if ref is not None:
            rr = graph_time([lambda: ref.ggml_moe_a8_vec(xs, c["w13"], tid, top_k, t, 2 * inter, tk)] * 2, reps=3)
            rv.update(us_reference=rr * 1e6)
        print(json.dumps(rv), flush=True)


def sweep_dequant(ref):
    import torch

    from gguf_b200 import capi, synth

    hbm, _, _ = peaks()
    for (t, n, k) in [(Q4_K, 14336, 4096), (Q4_0, 14336, 4096), (Q8_0, 14336, 4096), (Q6_K, 37888, 3584),
                      (IQ4_XS, 37888, 3584), (IQ2_XXS, 28672, 8192)]:
        wb, ws = rolled_copies(t, n, k, 200e6)
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
        x = torch.from_numpy(synth.make_activation(m, k, seed=0)).to("cuda")
        tq = graph_time([lambda: capi.quantize_q8_1(x)] * 8)
        moved = m * k * 2 + m * k // 32 * 36
        print(json.dumps(dict(op="quantize_q8_1 (36-byte blocks)", M=m, K=k, us=tq * 1e6, GBs=moved / tq / 1e9)), flush=True)


def run_sweep(what: str, with_ref: bool):
    ref = load_ref_cuda() if with_ref else None
    if with_ref and ref is None:
        raise SystemExit("--ref needs oracle/_ref/_C_gguf_ref.so (python oracle/build_ref.py where the reference sources are)")
    {"gemv": sweep_gemv, "gemm": sweep_gemm, "moe": sweep_moe, "dequant": sweep_dequant}[what](ref)


def run_ncu_case(spec: str):
    """Six back-to-back calls of one entry point on distinct weight copies, nothing timed."""
    import torch

    from gguf_b200 import capi, synth

    op, t, n, k, m = spec.split(",")
    t, n, k, m = int(t), int(n), int(k), int(m)
    if op == "moe":   # the MoE configuration's gate/up GEMM (type, sizes fixed by moe_case)
        c = moe_case()
        s_, e_, n_ = c["ours"]
        for _ in range(4):
            capi.moe_a8(c["x1"], c["w13"], s_, e_, n_, c["t"], 2 * c["inter"], c["top_k"], c["tokens"])
        torch.cuda.synchronize()
        print("ncu case done, device status", capi.last_status())
        return
    base = synth.make_weight(t, n, k, seed=1)
    ws = [torch.from_numpy(base).to("cuda") for _ in range(6)]
    x = torch.from_numpy(synth.make_activation(m, k, seed=0)).to("cuda")
    fn = {"gemv": capi.mul_mat_vec_a8, "mmq": capi.mul_mat_a8, "dqmm": capi.dequant_matmul}.get(op)
    for w in ws:
        if op == "dequantize":
            capi.dequantize(w, t, n, k)
        else:
            fn(w, x, t, n)
    torch.cuda.synchronize()
    print("ncu case done, device status", capi.last_status())


# --------------------------------------------------------------------------------------------
# extras
# --------------------------------------------------------------------------------------------

def c5_extras(world, rank, dev, stream, reps=10):
    """The largest configuration, column-sharded over `world` GPUs: IQ2_XXS up (28672 x 8192) and
    down (8192 x 28672) projections, tokens/s = M / (t_up + t_down) with the gathers inside the
    time, for one activation vector (decode GEMV, packets) and for 128 rows (tensor-core GEMM,
    tiles stored into every rank's output + flags; NCCL all-gather variant next to it).  Ten
    row-rotated copies of each matrix (1.2 GB in all, > L2 per rank at every N) are walked per
    step.  Parity: every rank compares copy 0 with the unsharded result it computes itself."""
    import torch
    import torch.distributed as dist

    from gguf_b200 import capi, synth, tp

    n_up, k_up = 28672, 8192
    copies = 10
    t = IQ2_XXS
    full_up = torch.from_numpy(synth.make_weight(t, n_up, k_up, seed=500)).to(dev)
    full_dn = torch.from_numpy(synth.make_weight(t, k_up, n_up, seed=501)).to(dev)
    sh_up, sh_dn = tp.shard_rows(full_up, rank, world), tp.shard_rows(full_dn, rank, world)
    w_up = [sh_up] + [sh_up.roll(c, 0).contiguous() for c in range(1, copies)]
    w_dn = [sh_dn] + [sh_dn.roll(c, 0).contiguous() for c in range(1, copies)]
    out = {"workload": "IQ2_XXS 28672x8192 (up) and 8192x28672 (down), column-sharded over %d GPU(s), %d copies per step" % (world, copies),
           "weight_bytes_per_token_all_ranks": 2 * 60555264}
    rel = lambda a, b: float((a.float() - b.float()).norm() / b.float().norm())

    def timed(fn):
        with torch.cuda.stream(stream):
            for _ in range(2):
                fn()
            stream.synchronize()
            run = fn
            try:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    fn()
                run = g.replay
            except Exception:
                torch.cuda.synchronize()
            for _ in range(3):
                run()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(reps):
                run()
            e1.record(stream)
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
        tt = torch.tensor([e0.elapsed_time(e1) / 1e3 / reps], device=dev)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return float(tt.item())

    # ---- M = 1: decode chain up_c -> down_c -> up_{c+1} ... through packets -------------------
    x1 = torch.from_numpy(synth.make_activation(1, k_up, seed=9)).to(dev)
    s_dn, s_res = 2.0 ** -5, 2.0 ** -12
    gv = tp.FusedGatherGemv(n_up, 2 * copies, torch.float16, dev)
    last = torch.empty((1, k_up), dtype=torch.float16, device=dev)

    def decode_step():
        for c in range(copies):
            gv(2 * c, w_up[c], x1, t, add_slot=(2 * c - 1) if c else -1, add_scale=s_res)   # x + s * down_{c-1}
            gv(2 * c + 1, w_dn[c], None, t, add_slot=2 * c, add_scale=s_dn)                 # s * up_c
        gv.gathered(2 * copies - 1, n=k_up, out=last)

    t1 = timed(decode_step)
    with torch.cuda.stream(stream):
        y_up = gv.gathered(0)
        y_dn = gv.gathered(1, n=k_up)
        want_up = capi.mul_mat_vec_a8(full_up, x1, t, n_up)
        want_dn = capi.mul_mat_vec_a8(full_dn, (s_dn * want_up.float()).half(), t, k_up)
        stream.synchronize()
        p1 = max(rel(y_up, want_up), rel(y_dn, want_dn))
        exact1 = bool(torch.equal(y_up, want_up) and torch.equal(y_dn, want_dn))
    out["m1"] = {"tokens_per_s": copies / t1, "us_per_token": t1 / copies * 1e6,
                 "weight_GBs_all_ranks": copies * 2 * 60555264 / t1 / 1e9,
                 "path": "gemv1 kernel, packets into every rank's memory, next call's quantizer reads them",
                 "rel_l2_vs_unsharded": p1, "bit_equal_to_unsharded": exact1}
    del gv

    # ---- M = 128: up -> wait -> down (reads the gathered up output) -> wait --------------------
    m = 128
    xm = torch.from_numpy(synth.make_activation(m, k_up, seed=10)).to(dev)
    mm = tp.FusedGatherMatmul(m, n_up, 2, torch.float16, dev)

    def prefill_step():
        for c in range(copies):
            yu = mm(0, capi.OP_DEQUANT_MATMUL, w_up[c], xm, t)
            mm(1, capi.OP_DEQUANT_MATMUL, w_dn[c], yu, t)

    t128 = timed(prefill_step)
    with torch.cuda.stream(stream):
        yu = mm(0, capi.OP_DEQUANT_MATMUL, w_up[0], xm, t).clone()
        yd = mm(1, capi.OP_DEQUANT_MATMUL, w_dn[0], yu, t).clone()
        want_u = capi.dequant_matmul(full_up, xm, t, n_up)
        want_d = capi.dequant_matmul(full_dn, want_u, t, k_up)
        stream.synchronize()
        p128 = max(rel(yu, want_u), rel(yd, want_d))
    flops = 2.0 * m * n_up * k_up * 2
    _, tf, _ = peaks()
    out["m128"] = {"tokens_per_s": m * copies / t128, "us_per_pair": t128 / copies * 1e6,
                   "tflops_all_ranks": flops * copies / t128 / 1e12, "frac_of_measured_16bit_peak_all_ranks": flops * copies / t128 / 1e12 / (tf * world),
                   "path": "tcgen05 dequant-GEMM, tiles stored into every rank's output over NVLink, flag wait",
                   "rel_l2_vs_unsharded": p128}
    if world > 1:   # the plain collective next to it: local GEMM + NCCL all-gather + column reassembly
        def prefill_nccl():
            for c in range(copies):
                yu = tp.gather_columns(capi.dequant_matmul(w_up[c], xm, t, n_up // world))
                tp.gather_columns(capi.dequant_matmul(w_dn[c], yu, t, k_up // world))

        tn = timed(prefill_nccl)
        out["m128"]["nccl_all_gather_variant"] = {"tokens_per_s": m * copies / tn, "us_per_pair": tn / copies * 1e6}
    out["device_status"] = capi.last_status()
    del mm, w_up, w_dn, full_up, full_dn
    torch.cuda.empty_cache()
    return out


def n1_extras(dev, stream, weights):
    """Single-GPU secondary figures: tensor-core GEMM and MoE throughput against the measured
    16-bit tensor peak (and twice it, as a stand-in for the int8 peak that was not measured), and
    the reference's own CUDA kernels timed on the same inputs in the same process."""
    import torch

    from gguf_b200 import capi, synth
    from vllm_gguf_plugin import ops

    hbm, tf, _ = peaks()
    ref = load_ref_cuda()
    extras = {}

    def gemm_fig(name, op, t, n, k, m, ws):
        x = torch.from_numpy(synth.make_activation(m, k, seed=0)).to(dev)
        fn = capi.mul_mat_a8 if op == "mmq" else capi.dequant_matmul
        tm = graph_time([lambda w=w: fn(w, x, t, n) for w in ws])
        flops = 2.0 * m * n * k
        r = {"us_per_call": tm * 1e6, "tflops": flops / tm / 1e12, "bound": "tensor (fp16 operands, fp32 accumulate)",
             "frac_of_measured_16bit_peak": flops / tm / 1e12 / tf, "frac_of_2x_that_as_int8_proxy": flops / tm / 1e12 / (2 * tf),
             "includes": "activation quantization + tcgen05 GEMM" if op == "mmq" else "tcgen05 dequant-GEMM on fp16 activations"}
        if ref is not None:
            if op == "mmq":
                tr = graph_time([lambda w=w: ref.ggml_mul_mat_a8(w, x, t, n) for w in ws[:3]], reps=2, warm=1)
            else:
                tr = graph_time([lambda w=w: x @ ref.ggml_dequantize(w, t, n, k, torch.float16).T for w in ws[:3]], reps=2, warm=1)
            r.update(reference_cuda_us_per_call=tr * 1e6, speedup_vs_reference_cuda=tr / tm)
        extras[name] = r

    gemm_fig("prefill_gemm_q4k_m512_14336x4096", "mmq", Q4_K, 14336, 4096, 512, weights[0])
    gemm_fig("prefill_gemm_q4k_m512_4096x14336", "mmq", Q4_K, 4096, 14336, 512, weights[1])
    _, ws = rolled_copies(Q6_K, 37888, 3584, 300e6, dev=dev)
    gemm_fig("prefill_gemm_q6k_m256_37888x3584", "mmq", Q6_K, 37888, 3584, 256, ws)
    del ws
    _, ws = rolled_copies(IQ4_XS, 37888, 3584, 300e6, dev=dev)
    gemm_fig("prefill_dequant_gemm_iq4xs_m256_37888x3584", "dqmm", IQ4_XS, 37888, 3584, 256, ws)
    del ws
    torch.cuda.empty_cache()
    extras["moe_q4_0_olmoe_256_tokens"] = moe_times(moe_case(dev), ref)

    # the reference's own decode kernel on the headline workload (same 32 weight copies, same graph method)
    if ref is not None:
        xs = [torch.from_numpy(synth.make_activation(1, k, seed=si)).to(dev) for si, (_, k) in enumerate(SHAPES)]
        calls_ref = [lambda w=w, si=si: ref.ggml_mul_mat_vec_a8(w, xs[si], Q4_K, SHAPES[si][0]) for si in range(2) for w in weights[si]]
        calls_our = [lambda w=w, si=si: ops.ggml_mul_mat_vec_a8(w, xs[si], Q4_K, SHAPES[si][0]) for si in range(2) for w in weights[si]]
        tr, to = graph_time(calls_ref, reps=10), graph_time(calls_our, reps=10)
        b = 33030144
        extras["reference_cuda_kernels_headline_workload"] = {
            "what": "the reference plugin's own CUDA extension (compiled for sm_100a from its sources) on the headline workload, "
                    "timed in this process after the timed regions above",
            "reference_us_per_call": tr * 1e6, "reference_GBs": b / tr / 1e9, "ours_us_per_call": to * 1e6, "ours_GBs": b / to / 1e9,
            "speedup": tr / to}
    else:
        extras["reference_cuda_kernels_headline_workload"] = {"unavailable": "oracle/_ref/_C_gguf_ref.so not built"}

    # ---- the linear layers of one Llama-3-8B decode step, batch 1 -----------------------------
    # 32 layers x (qkv 6144x4096, o 4096x4096, gate+up 28672x4096, down 4096x14336), Q4_K;
    # four seeded layer copies (488 MB > L2) are walked round-robin inside one CUDA graph.
    layer_shapes = [(6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336)]
    n_layers, n_copies = 32, 4
    lw = [[torch.from_numpy(synth.make_weight(Q4_K, n, k, seed=7000 + 10 * c + j)).to(dev)
           for j, (n, k) in enumerate(layer_shapes)] for c in range(n_copies)]
    lx = {k: torch.randn(1, k, device=dev, dtype=torch.float16) for k in (4096, 14336)}
    calls = [lambda layer=layer, j=j, n=n, k=k: ops.ggml_mul_mat_vec_a8(lw[layer % n_copies][j], lx[k], Q4_K, n)
             for layer in range(n_layers) for j, (n, k) in enumerate(layer_shapes)]
    t_tok = graph_time(calls, reps=20) * len(calls)
    layer_bytes = sum(n * (k // 256) * 144 for n, k in layer_shapes)
    extras["decode_linear_layers_llama3_8b_q4k_batch1"] = {
        "ms_per_token": t_tok * 1e3, "tokens_per_s": 1.0 / t_tok, "weight_GBs": n_layers * layer_bytes / t_tok / 1e9,
        "frac_of_measured_hbm": n_layers * layer_bytes / t_tok / 1e9 / hbm,
        "covers": "the 128 quantized GEMVs (with their activation quantizers) of one decode step; attention, norms, "
                  "embedding and lm_head are outside this path"}
    del lw
    torch.cuda.empty_cache()
    return extras


# --------------------------------------------------------------------------------------------
# main
# --------------------------------------------------------------------------------------------

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--sweep", default=None, choices=["gemv", "gemm", "moe", "dequant"])
    ap.add_argument("--ref", action="store_true", help="with --sweep: also time the reference's own CUDA kernels")
    ap.add_argument("--ncu-case", default=None,
                    help="op,type,N,K,M: run six plain calls of one kernel and exit (a small target for ncu captures)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)
    if args.ncu_case:
        return run_ncu_case(args.ncu_case)
    if args.sweep:
        return run_sweep(args.sweep, args.ref)

    import torch
    import torch.distributed as dist

    from gguf_b200 import capi, synth
    from vllm_gguf_plugin import ops  # raises if the CUDA extension is missing

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # plain peer stores only
        dist.init_process_group("nccl", device_id=dev)
    g = world
    warmup = max(args.warmup, 3)
    hbm_peak, tf_peak, which_peak = peaks()

    # ---- workload: COPIES seeded copies of each shape; rank r keeps its row slice -------------
    weights = []
    total_bytes = 0
    for si, (n_rows, k) in enumerate(SHAPES):
        assert n_rows % g == 0
        lo, hi = rank * n_rows // g, (rank + 1) * n_rows // g
        ws = []
        for c in range(COPIES):
            w = synth.make_weight(Q4_K, n_rows, k, seed=1000 * si + c)
            total_bytes += w.nbytes
            ws.append(torch.from_numpy(np.ascontiguousarray(w[lo:hi])).to(dev))
        weights.append(ws)
    calls_per_step = COPIES * len(SHAPES)
    kmax = max(k for _, k in SHAPES)
    # activations ("seeds"): row 2c = up call c (first 4096 values used), row 2c+1 = down call c
    seeds_np = np.zeros((calls_per_step, kmax), dtype=np.float16)
    for c in range(COPIES):
        seeds_np[2 * c, :SHAPES[0][1]] = synth.make_activation(1, SHAPES[0][1], seed=100 + c)[0]
        seeds_np[2 * c + 1, :SHAPES[1][1]] = synth.make_activation(1, SHAPES[1][1], seed=200 + c)[0]
    seeds_host = torch.from_numpy(seeds_np).pin_memory()
    seeds = seeds_host.to(dev)
    x_of = lambda si, c: seeds[2 * c + si, :SHAPES[si][1]].view(1, -1)
    outs_host = [torch.empty((COPIES, n_rows), dtype=torch.float16).pin_memory() for (n_rows, _) in SHAPES]
    outs_dev = [torch.empty((COPIES, n_rows), dtype=torch.float16, device=dev) for (n_rows, _) in SHAPES]
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())

    fused = None
    if g > 1:
        from gguf_b200.tp import FusedGatherGemv

        fused = FusedGatherGemv(max(n for n, _ in SHAPES), calls_per_step, torch.float16, dev)
        last_out = torch.empty((1, SHAPES[1][0]), dtype=torch.float16, device=dev)
    ys = [[None] * COPIES for _ in SHAPES]

    def step_body():
        """One pass: every weight copy of both shapes meets its activation vector once."""
        if fused is None:
            for si, (n_rows, k) in enumerate(SHAPES):
                for c in range(COPIES):
                    ys[si][c] = ops.ggml_mul_mat_vec_a8(weights[si][c], x_of(si, c), Q4_K, n_rows)
            return
        # N > 1: one dependent chain; slot c = up_c, slot COPIES + c = down_c
        seeds.neg_()
        for c in range(COPIES):
            fused(c, weights[0][c], x_of(0, c), Q4_K, add_slot=(COPIES + c - 1) if c else -1, add_scale=CHAIN_SCALE)
            fused(COPIES + c, weights[1][c], x_of(1, c), Q4_K, add_slot=c, add_scale=CHAIN_SCALE)
        fused.gathered(2 * COPIES - 1, n=SHAPES[1][0], out=last_out)   # the step ends when the last gather is complete here

    # warm up eagerly, then capture the step in a CUDA graph
    graph, use_graph = None, True
    with torch.cuda.stream(stream):
        for _ in range(2 if g > 1 else 3):   # (an even number of sign flips)
            step_body()
        stream.synchronize()
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                step_body()
        except Exception as exc:
            use_graph, graph = False, None
            print(f"[bench] graph capture failed ({type(exc).__name__}: {exc}); running eagerly", file=sys.stderr)
    torch.cuda.synchronize()

    def run_step():
        if use_graph:
            graph.replay()
        else:
            step_body()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        """CUDA-event time of `steps` calls of fn on `stream`, max over ranks, seconds."""
        with torch.cuda.stream(stream):
            for _ in range(warmup):
                fn()
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(steps):
                fn()
            e1.record(stream)
            barrier()
        t = torch.tensor([e0.elapsed_time(e1) / 1e3], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    with ClockSampler(local) as clocks:
        clocks.mark()
        t_dev = timed(run_step, args.steps)

        # ---- e2e: host activations in, host outputs out, every step -------------------------
        def e2e_step():
            seeds.copy_(seeds_host, non_blocking=True)
            run_step()
            if fused is None:
                for si in range(len(SHAPES)):
                    torch.cat(ys[si], dim=0, out=outs_dev[si])
            else:
                fused.gathered(0, COPIES, n=SHAPES[0][0], out=outs_dev[0])
                fused.gathered(COPIES, COPIES, n=SHAPES[1][0], out=outs_dev[1])
            for si in range(len(SHAPES)):
                outs_host[si].copy_(outs_dev[si], non_blocking=True)
            stream.synchronize()  # the caller reads the result every step

        t_e2e = timed(e2e_step, args.steps)

        # ---- the GEMV kernel alone: activations pre-quantized, graph of back-to-back launches --
        with torch.cuda.stream(stream):
            prepared = [[capi.gemv_prepare(x_of(si, c), Q4_K) for c in range(COPIES)] for si in range(len(SHAPES))]
            ybuf = [torch.empty((1, n_rows // g), dtype=torch.float16, device=dev) for (n_rows, _) in SHAPES]
            stream.synchronize()
        t_k = graph_time([lambda si=si, c=c: capi.gemv_prepared(weights[si][c], prepared[si][c], Q4_K, 1, SHAPES[si][0] // g, SHAPES[si][1], out=ybuf[si])
                          for si in range(len(SHAPES)) for c in range(COPIES)], reps=max(args.steps // 4, 10), warm=warmup)
    bytes_per_launch = total_bytes / g / calls_per_step
    achieved = bytes_per_launch / t_k / 1e9
    roof = {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
            "traffic": 33104128 // g,
            "traffic_source": "constant: dram__bytes_read.sum + dram__bytes_write.sum of one launch on a 33 MB matrix from an ncu "
                              "capture of this kernel (not measured in this run); divided by the number of ranks",
            "peak_source": which_peak, "kernel": "gemv1_kernel<Q4_K> (single-vector GEMV)",
            "us_per_launch": t_k * 1e6, "algorithmic_bytes_per_launch": bytes_per_launch}

    # ---- parity of what was just timed --------------------------------------------------------
    from oracle import cpu

    parity = {}
    with torch.cuda.stream(stream):
        run_step()
        stream.synchronize()
    if fused is None:
        w0 = synth.make_weight(Q4_K, SHAPES[0][0], SHAPES[0][1], seed=0)
        rows = np.linspace(0, SHAPES[0][0] - 1, 64).astype(np.int64)
        want, _ = cpu.matmul_a8(w0[rows], Q4_K, seeds[0:1, :SHAPES[0][1]].cpu().numpy(), "float16", mmq=False)
        got = ys[0][0].view(-1).float().cpu().numpy()[rows]
        parity["rel_l2_vs_oracle"] = float(np.linalg.norm(got - want[0]) / np.linalg.norm(want[0]))
        parity["checked"] = "64 rows spread over the first matrix"
    else:
        # whole gathered vectors as THIS rank holds them; rows from every rank's slice; the
        # activations of a checked call are rebuilt from the gathered vector it consumed
        with torch.cuda.stream(stream):
            y_up = fused.gathered(0, COPIES, n=SHAPES[0][0]).cpu().numpy()
            y_dn = fused.gathered(COPIES, COPIES, n=SHAPES[1][0]).cpu().numpy()
            stream.synchronize()
        sd = seeds.cpu().numpy()
        worst = 0.0
        for (si, c) in [(0, 0), (1, 0), (0, 1), (1, COPIES - 1), (0, COPIES - 1)]:
            n_rows, k = SHAPES[si]
            x = sd[2 * c + si, :k].astype(np.float32)
            prev = None if (si == 0 and c == 0) else (y_dn[c - 1] if si == 0 else y_up[c])
            if prev is not None:
                x = x + np.float32(CHAIN_SCALE) * prev[:k].astype(np.float32)
            x = x.astype(np.float16).reshape(1, k)
            w = synth.make_weight(Q4_K, n_rows, k, seed=1000 * si + c)
            per = n_rows // g
            rows = np.concatenate([r * per + np.linspace(0, per - 1, 16).astype(np.int64) for r in range(g)])
            want, _ = cpu.matmul_a8(w[rows], Q4_K, x, "float16", mmq=False)
            got = (y_up if si == 0 else y_dn)[c].astype(np.float32)[rows]
            worst = max(worst, float(np.linalg.norm(got - want[0]) / np.linalg.norm(want[0])))
        tw = torch.tensor([worst], device=dev)
        dist.all_reduce(tw, op=dist.ReduceOp.MAX)
        parity["rel_l2_vs_oracle"] = float(tw.item())
        parity["checked"] = ("max over ranks; on every rank 5 calls of the chain x 16 rows from EVERY rank's slice of the gathered "
                             "vector, activations rebuilt from the gathered vector the call consumed")

    # ---- N > 1: the same chain through NCCL (local GEMV + all_gather + torch residual add) ----
    extras = {}
    if g > 1:
        gathers = [torch.empty((COPIES, n_rows), dtype=torch.float16, device=dev) for (n_rows, _) in SHAPES]

        def nccl_step():
            seeds.neg_()
            for c in range(COPIES):
                for si in range(2):
                    n_rows, k = SHAPES[si]
                    x = x_of(si, c)
                    if si == 1 or c:
                        prev = gathers[0][c] if si == 1 else gathers[1][c - 1]
                        x = x + CHAIN_SCALE * prev[:k].view(1, -1)
                    y = ops.ggml_mul_mat_vec_a8(weights[si][c], x, Q4_K, n_rows // g)
                    dist.all_gather_into_tensor(gathers[si][c], y.view(-1))

        with torch.cuda.stream(stream):
            nccl_step()
            nccl_step()
            stream.synchronize()
            run_nccl = nccl_step
            try:
                ng = torch.cuda.CUDAGraph()
                with torch.cuda.graph(ng, stream=stream):
                    nccl_step()
                run_nccl = ng.replay
            except Exception:
                ng = None
                torch.cuda.synchronize()
        t_nccl = timed(run_nccl, max(args.steps // 4, 10))
        n_nccl = max(args.steps // 4, 10)
        extras["gather_latency"] = {
            "fused_packets_us_per_call": t_dev / args.steps / calls_per_step * 1e6,
            "nccl_all_gather_us_per_call": t_nccl / n_nccl / calls_per_step * 1e6,
            "gemv_kernel_alone_us_per_call": t_k * 1e6,
            "what": "one call = activation quantizer + GEMV on this rank's rows + all-gather, inside a chain of dependent calls"}
        if ng is not None:
            ng.reset()
        del gathers
    if not args.no_extras:
        extras["c5_iq2xxs_70b_mlp_column_sharded"] = c5_extras(world, rank, dev, stream)
        if world == 1:
            extras.update(n1_extras(dev, stream, weights))

    status = capi.last_status()

    def shutdown():
        """Leave without waiting on NCCL: a communicator that a live CUDA graph still references
        does not tear down, so the graph goes first and a watchdog ends the process regardless."""
        nonlocal graph
        if world == 1:
            return
        sys.stdout.flush()
        sys.stderr.flush()
        dog = threading.Timer(120.0, lambda: os._exit(0))
        dog.daemon = True
        dog.start()
        try:
            torch.cuda.synchronize()
            if graph is not None:
                graph.reset()
                graph = None
            # ranks leave together, idle: nobody exits while a peer may still touch mapped memory
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            os._exit(0)

    if rank != 0:
        shutdown()
        return

    cpu_base = None
    if not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        rows = SHAPES[0][0] // 2
        b, td, tm, _ = cpu_route_sample(rows, SHAPES[0][1], threads)
        cpu_base = {"value": b / (td + tm) / 1e9, "unit": "GB/s", "cores": threads, "kind": "reference",
                    "sample": f"{rows}x{SHAPES[0][1]} Q4_K rows (half of one matrix) once: gguf-py dequantize "
                              f"{td:.2f} s + torch fp32 matmul {tm * 1e3:.1f} ms",
                    "dequantize_s": td, "matmul_s": tm}

    value = total_bytes * args.steps / t_dev / 1e9
    e2e_val = total_bytes * args.steps / t_e2e / 1e9
    h2d = seeds_host.numel() * seeds_host.element_size()
    d2h = sum(o.numel() * o.element_size() for o in outs_host)
    parity["device_status"] = status
    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": g, "steps": args.steps, "warmup": warmup,
        "ms_per_step": t_dev / args.steps * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "int8", "data": "synthetic",
        "config": {"workload": "Q4_K GEMV M=1, Llama-3-8B shapes 14336x4096 and 4096x14336, 16 weight copies each per step",
                   "l2": "inputs larger than L2: 1.06 GB of weights per step, each copy read once",
                   "launch": "CUDA graph of one step" if use_graph else "eager",
                   "parallelism": (f"tp{g} column-sharded; all-gather fused into the GEMV (tagged packets stored into every rank's memory over "
                                   f"NVLink); the 32 calls of a step are one dependent chain") if g > 1 else "single GPU",
                   "weights_resident": True},
        "e2e": {"value": e2e_val, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": t_e2e / args.steps * 1e3},
        "gpu_launches": args.steps * (calls_per_step * 2 + (2 if g > 1 else 0)),
        "roofline": roof, "cpu_baseline": cpu_base, "clocks": clocks.summary(),
        "parity": parity,
        "extras": extras,
    }
    print(json.dumps(line), flush=True)
    shutdown()


if __name__ == "__main__":
    main()
