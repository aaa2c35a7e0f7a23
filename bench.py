"""Benchmark of the GGUF quantized-matmul hot path on B200.

    python bench.py --gpus N --steps K --warmup W            (this library)
    python bench.py --impl reference --gpus N --steps K ...  (the reference's CPU route)

Workload (N = 1): decode GEMV on Q4_K weights with the Llama-3-8B linear shapes
(K=4096 -> N=14336 and K=14336 -> N=4096, one fp16 activation vector, seeded synthetic
blocks).  One "step" is one pass over 16 independently generated copies of each of the two
matrices (32 GEMV calls, 1.06 GB of packed weights), so every call reads weights that have
been evicted from the 126 MB L2 since their last use.  A step is captured once in a CUDA
graph and replayed, as a serving engine does for decode.

Metric: quantized-weight bytes per second (GB/s), the numerator the GEMV roofline uses.
  value     inputs resident in HBM, whole step (activation quantization + GEMV kernels)
  e2e       the same step through the public operator API with HOST activations: pinned
            host -> device copy of the step's activations and device -> host read of its
            outputs inside the timed region
  roofline  the GEMV kernel alone (activations pre-quantized), algorithmic bytes / duration,
            against the measured copy bandwidth of MEASURED_PEAKS.json
  cpu_baseline  the reference's CPU route (gguf-py dequantize + torch fp32 matmul) on the
            host cores, on a bounded sample of the same workload

N > 1: the same matrices column-sharded over the ranks (rank r holds rows [r*N/g, (r+1)*N/g),
the reference's tensor-parallel slicing rule, quantization/params.py:227-236) with an NCCL
all-gather of the output slices after every GEMV; total work is fixed ("strong").
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

Q4_K = 12
SHAPES = [(14336, 4096), (4096, 14336)]  # (N rows, K) of the two Llama-3-8B linear shapes
COPIES = 16
METRIC = "quant GEMV HBM GB/s (quantized-weight bytes / s), Q4_K decode, Llama-3-8B linear shapes"


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        return self

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
        sm = [float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for r in self.rows if len(r) >= 6 for i in range(4) if r[2 + i].lower().startswith("active")})
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


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


def run_ncu_case(spec: str):
    """Six back-to-back calls of one entry point on distinct weight copies, nothing timed."""
    import torch

    from gguf_b200 import capi, synth

    op, t, n, k, m = spec.split(",")
    t, n, k, m = int(t), int(n), int(k), int(m)
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--ncu-case", default=None,
                    help="op,type,N,K,M: run six plain calls of one kernel and exit (a small target for ncu captures)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)
    if args.ncu_case:
        return run_ncu_case(args.ncu_case)

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
        dist.init_process_group("nccl", device_id=dev)
    g = world
    warmup = max(args.warmup, 3)

    # ---- workload: COPIES seeded copies of each shape; rank r keeps its row slice -------------
    weights, xs_host, xs_dev = [], [], []
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
        xh = torch.from_numpy(synth.make_activation(COPIES, k, seed=si)).pin_memory()
        xs_host.append(xh)
        xs_dev.append(torch.empty_like(xh, device=dev))
    for xd, xh in zip(xs_dev, xs_host):
        xd.copy_(xh)
    calls_per_step = COPIES * len(SHAPES)
    outs_full = [torch.empty((COPIES, n_rows), dtype=torch.float16, device=dev) for (n_rows, _) in SHAPES]
    outs_host = [torch.empty((COPIES, n_rows), dtype=torch.float16).pin_memory() for (n_rows, _) in SHAPES]
    gathers = [torch.empty((COPIES, g, n_rows // g), dtype=torch.float16, device=dev) for (n_rows, _) in SHAPES] if g > 1 else None
    # N > 1: the GEMV kernel stores its slice into every rank's output vector over NVLink and raises a
    # flag (no collective call per GEMV); NCCL all-gather only if peer-mapped memory cannot be set up
    fused = None
    if g > 1 and os.environ.get("GGUF_B200_BENCH_NCCL_GATHER", "0") != "1":
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # plain peer stores only
        try:
            from gguf_b200.tp import FusedGatherGemv

            fused = FusedGatherGemv(max(n for n, _ in SHAPES), len(SHAPES) * COPIES, torch.float16, dev)
        except Exception as exc:
            print(f"[bench] peer-mapped output unavailable ({type(exc).__name__}: {exc}); using NCCL all-gather", file=sys.stderr)
            fused = None

    ys = [[None] * COPIES for _ in SHAPES]

    def step_body():
        """One pass: every weight copy of both shapes meets its activation vector once."""
        for si, (n_rows, k) in enumerate(SHAPES):
            for c in range(COPIES):
                if fused is not None:
                    # a decode chain: each call's quantizer waits for the previous call's gather
                    slot = si * COPIES + c
                    ys[si][c] = fused(slot, weights[si][c], xs_dev[si][c:c + 1], Q4_K, wait_slot=slot - 1, wait=False)[:, :n_rows]
                    if slot == len(SHAPES) * COPIES - 1:
                        fused.wait(slot)
                    continue
                y = ops.ggml_mul_mat_vec_a8(weights[si][c], xs_dev[si][c:c + 1], Q4_K, n_rows // g)
                ys[si][c] = y
                if g > 1:
                    dist.all_gather_into_tensor(gathers[si][c], y.view(-1))

    # warm up eagerly (also lets NCCL set up), then capture the step in a CUDA graph
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    graph, use_graph = None, True
    with torch.cuda.stream(stream):
        for _ in range(3):
            step_body()
        stream.synchronize()
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                step_body()
        except Exception as exc:  # collectives that refuse capture: run eagerly and say so
            use_graph, graph = False, None
            print(f"[bench] graph capture failed ({type(exc).__name__}); running eagerly", file=sys.stderr)
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
        t_dev = timed(run_step, args.steps)

        # ---- e2e: host activations in, host outputs out, every step -------------------------
        def e2e_step():
            for xd, xh in zip(xs_dev, xs_host):
                xd.copy_(xh, non_blocking=True)
            run_step()
            for si in range(len(SHAPES)):
                if g > 1 and fused is None:
                    src = gathers[si].view(COPIES, -1)
                else:  # one gather kernel per shape: the step's outputs as one buffer
                    src = torch.cat(ys[si], dim=0, out=outs_full[si])
                outs_host[si].copy_(src, non_blocking=True)
            stream.synchronize()  # the caller reads the result every step

        t_e2e = timed(e2e_step, args.steps)

        # ---- the GEMV kernel alone: activations pre-quantized, graph of back-to-back launches --
        roof = None
        if rank == 0:
            with torch.cuda.stream(stream):
                prepared = [[capi.gemv_prepare(xs_dev[si][c:c + 1], Q4_K) for c in range(COPIES)] for si in range(len(SHAPES))]
                ybuf = [torch.empty((1, n_rows // g), dtype=torch.float16, device=dev) for (n_rows, _) in SHAPES]

                def gemv_only():
                    for si, (n_rows, k) in enumerate(SHAPES):
                        for c in range(COPIES):
                            capi.gemv_prepared(weights[si][c], prepared[si][c], Q4_K, 1, n_rows // g, k, out=ybuf[si])

                for _ in range(3):
                    gemv_only()
                stream.synchronize()
                kg = torch.cuda.CUDAGraph()
                with torch.cuda.graph(kg, stream=stream):
                    gemv_only()
                for _ in range(warmup):
                    kg.replay()
                stream.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                for _ in range(args.steps):
                    kg.replay()
                e1.record(stream)
                stream.synchronize()
                t_k = e0.elapsed_time(e1) / 1e3 / (args.steps * calls_per_step)
            peak, which = measured_peaks()
            bytes_per_launch = total_bytes / g / calls_per_step
            achieved = bytes_per_launch / t_k / 1e9
            roof = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                    # dram__bytes_read.sum + dram__bytes_write.sum of one launch, from the committed ncu capture
                    # (profiles/gemv1_q4k_llama8b_decode.md); both shapes move the same 33.03 MB of weights
                    "traffic": 33082500 // g, "peak_source": which, "kernel": "gemv1_kernel<Q4_K> (single-vector GEMV)",
                    "us_per_launch": t_k * 1e6, "algorithmic_bytes_per_launch": bytes_per_launch}
    if world > 1:
        dist.barrier()

    # ---- secondary figure (N = 1 only): the prefill GEMM of the same configuration, M = 512 -----
    extras = None
    if world == 1:
        with torch.cuda.stream(stream):
            xm = torch.randn(512, SHAPES[0][1], device=dev, dtype=torch.float16)
            for c in range(3):
                capi.mul_mat_a8(weights[0][c], xm, Q4_K, SHAPES[0][0])
            stream.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for c in range(COPIES):
                capi.mul_mat_a8(weights[0][c], xm, Q4_K, SHAPES[0][0])
            e1.record(stream)
            stream.synchronize()
            t_mm = e0.elapsed_time(e1) / 1e3 / COPIES
        flops = 2.0 * 512 * SHAPES[0][0] * SHAPES[0][1]
        peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
        tf_peak = float(peaks.get("bf16_tflops", 1590.0))
        extras = {"prefill_gemm_q4k_m512_14336x4096": {
            "us_per_call": t_mm * 1e6, "tflops": flops / t_mm / 1e12, "bound": "tensor (fp16 operands, fp32 accumulate)",
            "frac_of_measured_16bit_peak": flops / t_mm / 1e12 / tf_peak, "frac_of_2x_that_as_int8_proxy": flops / t_mm / 1e12 / (2 * tf_peak),
            "includes": "q8_1 quantization of the 512x4096 activations + tcgen05 GEMM"}}

        # ---- secondary figure: the linear layers of one Llama-3-8B decode step, batch 1 -----------
        # 32 layers x (qkv 6144x4096, o 4096x4096, gate+up 28672x4096, down 4096x14336), Q4_K;
        # four seeded layer copies (488 MB > L2) are walked round-robin inside one CUDA graph.
        layer_shapes = [(6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336)]
        n_layers, n_copies = 32, 4
        with torch.cuda.stream(stream):
            lw = [[torch.from_numpy(synth.make_weight(Q4_K, n, k, seed=7000 + 10 * c + j)).to(dev)
                   for j, (n, k) in enumerate(layer_shapes)] for c in range(n_copies)]
            lx = {k: torch.randn(1, k, device=dev, dtype=torch.float16) for k in (4096, 14336)}

            def decode_step():
                for layer in range(n_layers):
                    for j, (n, k) in enumerate(layer_shapes):
                        ops.ggml_mul_mat_vec_a8(lw[layer % n_copies][j], lx[k], Q4_K, n)

            decode_step()
            stream.synchronize()
            dg = torch.cuda.CUDAGraph()
            with torch.cuda.graph(dg, stream=stream):
                decode_step()
            for _ in range(3):
                dg.replay()
            stream.synchronize()
            e0.record(stream)
            reps = 20
            for _ in range(reps):
                dg.replay()
            e1.record(stream)
            stream.synchronize()
            t_tok = e0.elapsed_time(e1) / 1e3 / reps
        layer_bytes = sum(n * (k // 256) * 144 for n, k in layer_shapes)
        extras["decode_linear_layers_llama3_8b_q4k_batch1"] = {
            "ms_per_token": t_tok * 1e3, "tokens_per_s": 1.0 / t_tok, "weight_GBs": n_layers * layer_bytes / t_tok / 1e9,
            "covers": "the 128 quantized GEMVs (with their activation quantizers) of one decode step; attention, norms, "
                      "embedding and lm_head are outside this path"}
        del lw

    status = capi.last_status()

    def shutdown():
        """Leave without waiting on NCCL: a communicator that a live CUDA graph still references
        does not tear down, so the graph goes first and a watchdog ends the process regardless."""
        nonlocal graph
        if world == 1:
            return
        sys.stdout.flush()
        sys.stderr.flush()
        import threading

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

    # parity spot check of what was just timed (host oracle, tiny: first 64 rows of one copy)
    from oracle import cpu

    w0 = synth.make_weight(Q4_K, SHAPES[0][0], SHAPES[0][1], seed=0)[:64]
    want, _ = cpu.matmul_a8(w0, Q4_K, xs_host[0][0:1].numpy(), "float16", mmq=False)
    got = (gathers[0][0].view(-1) if (g > 1 and fused is None) else ys[0][0].view(-1))[:64].float().cpu().numpy()
    rel = float(np.linalg.norm(got - want[0]) / np.linalg.norm(want[0]))

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
    h2d = sum(x.numel() * x.element_size() for x in xs_host)
    d2h = sum(o.numel() * o.element_size() for o in outs_host)
    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": g, "steps": args.steps, "warmup": warmup,
        "ms_per_step": t_dev / args.steps * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "int8", "data": "synthetic",
        "config": {"workload": "Q4_K GEMV M=1, Llama-3-8B shapes 14336x4096 and 4096x14336, 16 weight copies each per step",
                   "l2": "inputs larger than L2: 1.06 GB of weights per step, each copy read once",
                   "launch": "CUDA graph of one step" if use_graph else "eager",
                   "parallelism": (f"tp{g} column-sharded, all-gather fused into the GEMV (peer stores over NVLink + flags)" if fused is not None
                                   else f"tp{g} column-sharded + NCCL all-gather") if g > 1 else "single GPU",
                   "weights_resident": True},
        "e2e": {"value": e2e_val, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": t_e2e / args.steps * 1e3},
        "gpu_launches": args.steps * (calls_per_step * 2 + (1 if fused is not None else 0)),
        "roofline": roof, "cpu_baseline": cpu_base, "clocks": clocks.summary(),
        "parity": {"rel_l2_vs_oracle": rel, "device_status": status},
        "extras": extras,
    }
    print(json.dumps(line), flush=True)
    shutdown()


if __name__ == "__main__":
    main()
