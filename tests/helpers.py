"""Shared helpers of the test-suite."""
from __future__ import annotations

import ctypes
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
# block types with fused matmul kernels (GEMV for all of them)
TYPES = {"Q4_0": 2, "Q8_0": 8, "Q4_K": 12, "Q6_K": 14, "IQ2_XXS": 16, "IQ4_XS": 23,
         "Q4_1": 3, "Q5_0": 6, "Q5_1": 7, "Q5_K": 13, "IQ4_NL": 20,
         "IQ2_XS": 17, "IQ3_XXS": 18, "IQ1_S": 19, "IQ3_S": 21, "IQ2_S": 22, "IQ1_M": 29, "Q2_K": 10, "Q3_K": 11}
# ... of which the q8_1 tensor-core GEMM serves these (the others take the dequantize-matmul route)
MMQ_TYPES = {k: TYPES[k] for k in ("Q4_0", "Q8_0", "Q4_K", "Q6_K", "Q4_1", "Q5_0", "Q5_1", "Q5_K", "Q2_K", "Q3_K")}
# types served by the standalone dequantize only
DEQUANT_ONLY_TYPES: dict = {}   # (none left: every type of the reference's dispatch has a GEMV here)
# the tolerance the task states for matmul outputs against the reference's own kernels
REL_L2_TOL = 2e-3


def rel_l2(a, b) -> float:
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def bits(t):
    """Bit pattern view of a torch tensor (for exact comparisons)."""
    import torch

    return t.view(torch.int32 if t.dtype == torch.float32 else torch.int16)


def np_act(x_t):
    """torch activation tensor -> the numpy array the CPU oracle takes (+ its dtype name)."""
    import torch

    if x_t.dtype == torch.bfloat16:
        return x_t.view(torch.int16).cpu().numpy().view(np.uint16), "bfloat16"
    return x_t.cpu().numpy(), str(x_t.dtype).split(".")[1]


class RefCuda:
    """The reference plugin's own CUDA extension (oracle/_ref/_C_gguf_ref.so), when it was built.

    GPU parity tests use it as the authoritative comparison; they fall back to the CPU oracle
    alone when the file is absent."""

    def __init__(self):
        import torch

        so = ROOT / "oracle" / "_ref" / "_C_gguf_ref.so"
        self.available = so.exists()
        if self.available:
            torch.ops.load_library(str(so))
            self.ops = torch.ops._C_gguf_ref
            self.lib = ctypes.CDLL(str(so))

    def quantize_q8_1(self, X):
        import torch

        M, K = X.shape
        rb = (K + 511) // 512 * 512 // 32 * 36
        out = torch.zeros((M, rb), dtype=torch.uint8, device=X.device)
        code = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}[X.dtype]
        rc = self.lib.ref_quantize_q8_1(ctypes.c_void_p(X.data_ptr()), code, ctypes.c_void_p(out.data_ptr()), K, M,
                                        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        assert rc == 0
        return out
