"""Generate the committed golden fixtures of this directory.  Run from the repository root:

    python tests/golden/make_golden.py

Two fixtures, both produced by code that is NOT this repository's:

* golden_gguf_py.npz -- for each of the six block types a few seeded random blocks and the
  output of ``gguf.dequantize`` (gguf-py, the third-party definition of the formats that the
  reference's own kernel tests compare against, tests/test_kernels.py:77-99), plus
  ``x @ dequantize(W).T`` in float64 for a small activation matrix (the reference's CPU route).
* golden_routing.json -- which operator the reference's dispatcher
  ``_fused_mul_mat_gguf`` (vllm_gguf_plugin/quantization/linear.py:35-58) calls for each
  (type, batch, rows), recorded by importing the reference module from its checkout with its
  ``ops`` functions replaced by recorders.  Needs the reference checkout (GGUF_REFERENCE_ROOT) and
  vLLM; skipped if absent.
"""
from __future__ import annotations

import importlib
import os
import json
import sys
import types
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT / "vllm-gguf-plugin-prism_b200"))
sys.path.insert(0, str(ROOT))

TYPES = {"Q4_0": 2, "Q8_0": 8, "Q4_K": 12, "Q6_K": 14, "IQ2_XXS": 16, "IQ4_XS": 23,
         "Q4_1": 3, "Q5_0": 6, "Q5_1": 7, "Q5_K": 13, "IQ4_NL": 20,
         "IQ2_XS": 17, "IQ3_XXS": 18, "IQ1_S": 19, "IQ3_S": 21, "IQ2_S": 22, "IQ1_M": 29, "Q2_K": 10, "Q3_K": 11}
# dequantize fixtures only (no fused matmul for these in this library)
DEQUANT_ONLY: dict = {}


def gguf_py_fixture():
    import gguf
    from gguf_b200 import synth

    out = {}
    for name, t in {**TYPES, **DEQUANT_ONLY}.items():
        n, k = 6, 512
        w = synth.make_weight(t, n, k, seed=40 + t)
        wd = gguf.dequantize(w, gguf.GGMLQuantizationType(t)).astype(np.float32)
        x = synth.make_activation(3, k, seed=7, dtype=np.float16)
        out[f"w_{name}"] = w
        out[f"dq_{name}"] = wd
        out[f"x_{name}"] = x
        out[f"y_{name}"] = x.astype(np.float64) @ wd.astype(np.float64).T
    np.savez_compressed(HERE / "golden_gguf_py.npz", **out)
    print("wrote golden_gguf_py.npz")


def routing_fixture(ref_root=None):
    from oracle import reference_root

    ref_root = ref_root or reference_root()
    if ref_root is None:
        print("reference checkout absent: golden_routing.json not regenerated")
        return
    import torch

    # import the reference's quantization.linear without running its package __init__
    pkg = types.ModuleType("vllm_gguf_plugin")
    pkg.__path__ = [str(ref_root / "vllm_gguf_plugin")]
    saved = {k: sys.modules.pop(k) for k in list(sys.modules) if k == "vllm_gguf_plugin" or k.startswith("vllm_gguf_plugin.")}
    sys.modules["vllm_gguf_plugin"] = pkg
    try:
        ops = importlib.import_module("vllm_gguf_plugin.ops")
        linear = importlib.import_module("vllm_gguf_plugin.quantization.linear")
        calls = []

        def rec(name, shape_fn):
            def f(*a, **kw):
                calls.append(name)
                return shape_fn(*a)
            return f

        ops.ggml_mul_mat_vec_a8 = rec("ggml_mul_mat_vec_a8", lambda W, X, t, row: torch.zeros(X.shape[0], row))
        ops.ggml_mul_mat_a8 = rec("ggml_mul_mat_a8", lambda W, X, t, row: torch.zeros(X.shape[0], row))
        ops.ggml_dequantize = rec("ggml_dequantize", lambda W, t, m, n, dt: torch.zeros(m, n, dtype=dt))
        table = []
        from gguf_b200 import synth

        for name, t in TYPES.items():
            bs, ts = synth.QUANT_SIZES[t]
            for rows in (4096, 5120, 5121, 14336):
                for m in (0, 1, 2, 3, 6, 7, 8, 9, 16, 17, 64, 512):
                    calls.clear()
                    w = torch.zeros(rows, 256 // bs * ts, dtype=torch.uint8)
                    x = torch.zeros(m, 256, dtype=torch.float16)
                    linear._fused_mul_mat_gguf(x, w, t)
                    table.append({"type": t, "rows": rows, "m": m, "calls": list(calls)})
        (HERE / "golden_routing.json").write_text(json.dumps(table))
        print("wrote golden_routing.json:", len(table), "cases")
    finally:
        for k in [k for k in sys.modules if k == "vllm_gguf_plugin" or k.startswith("vllm_gguf_plugin.")]:
            del sys.modules[k]
        sys.modules.update(saved)


if __name__ == "__main__":
    gguf_py_fixture()
    routing_fixture()
