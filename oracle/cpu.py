"""ctypes wrapper of oracle/gguf_oracle.c plus the reference's CPU route (gguf-py + fp32 matmul).

Test infrastructure only.  The C file is compiled on first use into
oracle/_build/libgguf_oracle.so with gcc (no fast-math, no fp contraction).
"""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
_SO = HERE / "_build" / "libgguf_oracle.so"
_lib = None

DT = {"float32": 0, "float16": 1, "bfloat16": 2}
TYPES = {"Q4_0": 2, "Q8_0": 8, "Q4_K": 12, "Q6_K": 14, "IQ2_XXS": 16, "IQ4_XS": 23}


def build(force: bool = False) -> Path:
    src = HERE / "gguf_oracle.c"
    hdr = HERE.parent / "include" / "gguf_b200_iq_tables.h"
    if force or not _SO.exists() or _SO.stat().st_mtime < max(src.stat().st_mtime, hdr.stat().st_mtime):
        _SO.parent.mkdir(exist_ok=True)
        subprocess.check_call(["gcc", "-O2", "-ffp-contract=off", "-fno-fast-math", "-shared", "-fPIC",
                               str(src), "-o", str(_SO), "-lm"])
    return _SO


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(str(build()))
        _lib.oracle_q8_1_row_bytes.restype = ctypes.c_int64
        _lib.oracle_q8_1_row_bytes.argtypes = [ctypes.c_int64]
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p) if a is not None else None


def type_size(t: int) -> int:
    return lib().oracle_type_size(int(t))


def block_size(t: int) -> int:
    return lib().oracle_block_size(int(t))


def _out_array(n: int, dtype: str):
    return np.empty(n, dtype=np.float32 if dtype == "float32" else np.uint16)


def as_float(bits: np.ndarray, dtype: str) -> np.ndarray:
    """Raw output of the oracle (uint16 bit patterns for 16-bit dtypes) -> float32 values."""
    if dtype == "float32":
        return bits
    if dtype == "float16":
        return bits.view(np.float16).astype(np.float32)
    return (bits.astype(np.uint32) << 16).view(np.float32)


def dequantize(w: np.ndarray, t: int, n_elems: int, dtype: str = "float16", q4k_contract: int = 1) -> np.ndarray:
    """Bit pattern of ggml_dequantize's output (uint16 for float16/bfloat16, float32 otherwise)."""
    w = np.ascontiguousarray(w, dtype=np.uint8)
    out = _out_array(n_elems, dtype)
    rc = lib().oracle_dequantize(_p(w), int(t), _p(out), DT[dtype], ctypes.c_int64(n_elems), int(q4k_contract))
    assert rc == 0
    return out


def _act(x: np.ndarray, dtype: str) -> np.ndarray:
    """Activations as the raw array the C side reads: float32, float16, or bfloat16 bits (uint16)."""
    if dtype == "float32":
        return np.ascontiguousarray(x, dtype=np.float32)
    if dtype == "float16":
        return np.ascontiguousarray(x, dtype=np.float16)
    assert x.dtype == np.uint16, "pass bfloat16 activations as uint16 bit patterns"
    return np.ascontiguousarray(x)


def quantize_q8_1(x: np.ndarray, dtype: str = "float16") -> np.ndarray:
    """[M,K] activations -> uint8 [M, Kpad/32*36] in the block_q8_1 layout (d, sum, 32 x int8)."""
    x = _act(x, dtype)
    M, K = x.shape
    rb = lib().oracle_q8_1_row_bytes(K)
    out = np.empty((M, rb), dtype=np.uint8)
    rc = lib().oracle_quantize_q8_1(_p(x), DT[dtype], _p(out), ctypes.c_int64(M), ctypes.c_int64(K))
    assert rc == 0
    return out


def matmul_a8(w: np.ndarray, t: int, x: np.ndarray, dtype: str = "float16", mmq: bool = False):
    """(unrounded float64 [M,N], output bits in `dtype`) of ggml_mul_mat_vec_a8 (mmq=False) / ggml_mul_mat_a8."""
    w = np.ascontiguousarray(w, dtype=np.uint8)
    N = w.shape[0]
    M, K = x.shape
    xq = quantize_q8_1(x, dtype)
    y64 = np.empty((M, N), dtype=np.float64)
    out = _out_array(M * N, dtype)
    rc = lib().oracle_matmul_a8(_p(w), int(t), _p(xq), _p(y64), _p(out), DT[dtype], ctypes.c_int64(M),
                                ctypes.c_int64(N), ctypes.c_int64(K), int(bool(mmq)))
    assert rc == 0
    return y64, out.reshape(M, N)


def moe_a8(w: np.ndarray, t: int, x: np.ndarray, sorted_ids: np.ndarray, expert_ids: np.ndarray, n_post_pad: int,
           block: int, top_k: int, tokens: int, dtype: str = "float16"):
    w = np.ascontiguousarray(w, dtype=np.uint8)
    E, N, rowb = w.shape
    K = x.shape[1]
    xq = quantize_q8_1(x, dtype)
    sorted_ids = np.ascontiguousarray(sorted_ids, dtype=np.int32)
    expert_ids = np.ascontiguousarray(expert_ids, dtype=np.int32)
    rows = tokens * top_k
    y64 = np.empty((rows, N), dtype=np.float64)
    out = _out_array(rows * N, dtype)
    rc = lib().oracle_moe_a8(_p(w), int(t), _p(xq), _p(y64), _p(out), DT[dtype], _p(sorted_ids),
                             ctypes.c_int64(sorted_ids.size), _p(expert_ids), ctypes.c_int32(int(n_post_pad)),
                             int(block), ctypes.c_int64(N * rowb), ctypes.c_int64(tokens), ctypes.c_int64(top_k),
                             ctypes.c_int64(N), ctypes.c_int64(K))
    assert rc == 0
    return y64, out.reshape(rows, N)


def moe_a8_vec(w: np.ndarray, t: int, x: np.ndarray, topk_ids: np.ndarray, top_k: int, tokens: int,
               dtype: str = "float16"):
    w = np.ascontiguousarray(w, dtype=np.uint8)
    E, N, rowb = w.shape
    K = x.shape[1]
    xq = quantize_q8_1(x, dtype)
    ids = np.ascontiguousarray(topk_ids, dtype=np.int32).reshape(-1)
    rows = tokens * top_k
    y64 = np.empty((rows, N), dtype=np.float64)
    out = _out_array(rows * N, dtype)
    rc = lib().oracle_moe_a8_vec(_p(w), int(t), _p(xq), _p(y64), _p(out), DT[dtype], _p(ids),
                                 ctypes.c_int64(tokens), ctypes.c_int64(top_k), ctypes.c_int64(N), ctypes.c_int64(K))
    assert rc == 0
    return y64, out.reshape(rows, N)


def dense_matmul(wd: np.ndarray, x: np.ndarray, dtype: str = "float16") -> np.ndarray:
    """float64 x @ wd.T with wd = dequantized weights (the dequantize-then-matmul route)."""
    wd = np.ascontiguousarray(wd, dtype=np.float32)
    x = _act(x, dtype)
    N, K = wd.shape
    M = x.shape[0]
    y64 = np.empty((M, N), dtype=np.float64)
    rc = lib().oracle_dense_matmul(_p(wd), _p(x), DT[dtype], _p(y64), ctypes.c_int64(M), ctypes.c_int64(N),
                                   ctypes.c_int64(K))
    assert rc == 0
    return y64


# ---- the reference's CPU route: gguf-py numpy dequantize + torch fp32 matmul ----------

def gguf_py_dequantize(w: np.ndarray, t: int) -> np.ndarray:
    """gguf.dequantize (gguf-py, the third-party package the reference's tests compare with)."""
    import gguf

    return gguf.dequantize(np.ascontiguousarray(w, dtype=np.uint8), gguf.GGMLQuantizationType(int(t)))


def cpu_route(w: np.ndarray, t: int, x_f32):
    """x @ dequantize(W).T in fp32 on the host cores (torch uses all threads it is given)."""
    import torch

    wd = torch.from_numpy(gguf_py_dequantize(w, t))
    return x_f32 @ wd.T
