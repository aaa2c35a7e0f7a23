"""ctypes binding of the C-ABI (include/gguf_b200.h) for callers that hold torch tensors.

This is the thinnest possible host layer: torch provides device memory and the current
stream, every computation is one call into ``libgguf_b200.so``.  The parity tests call the
kernels through this module so that what they exercise is the exported C interface itself.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

import torch

_LIB_PATH = Path(__file__).resolve().parent.parent / "vllm_gguf_plugin" / "libgguf_b200.so"
_lib = None

F32, F16, BF16 = 0, 1, 2
OP_GEMV, OP_MMQ, OP_MOE, OP_MOE_VEC, OP_DEQUANT_MATMUL = range(5)
_F = ctypes.c_float
_DT = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}

# name -> (restype, argtypes); mirrors include/gguf_b200.h one to one
_P, _I, _L = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64
SIGNATURES = {
    "gguf_b200_error_string": (ctypes.c_char_p, [_I]),
    "gguf_b200_version": (ctypes.c_char_p, []),
    "gguf_b200_type_size": (_I, [_I]),
    "gguf_b200_block_size": (_I, [_I]),
    "gguf_b200_q8_1_row_bytes": (_L, [_L]),
    "gguf_b200_quantize_q8_1": (_I, [_P, _I, _P, _L, _L, _P]),
    "gguf_b200_dequantize": (_I, [_P, _I, _P, _I, _L, _P]),
    "gguf_b200_dequantize_rows": (_I, [_P, _I, _P, _L, _L, _L, _P, _I, _P]),
    "gguf_b200_workspace_bytes": (_L, [_I, _I, _L, _L, _L]),
    "gguf_b200_mul_mat_vec_a8": (_I, [_P, _P, _P, _P, _L, _I, _I, _L, _L, _L, _P]),
    "gguf_b200_gemv_prepare": (_I, [_P, _I, _P, _L, _I, _L, _L, _P]),
    "gguf_b200_gemv_prepared": (_I, [_P, _P, _P, _I, _I, _L, _L, _L, _P]),
    "gguf_b200_mul_mat_a8": (_I, [_P, _P, _P, _P, _L, _I, _I, _L, _L, _L, _P]),
    "gguf_b200_dequant_matmul": (_I, [_P, _P, _P, _P, _L, _I, _I, _L, _L, _L, _P]),
    "gguf_b200_moe_a8": (_I, [_P, _P, _P, _P, _L, _P, _P, _P, _L, _L, _L, _I, _I, _L, _L, _L, _L, _P]),
    "gguf_b200_fused_moe_workspace_bytes": (_L, [_I, _I, _I, _L, _L, _L, _L, _L]),
    "gguf_b200_fused_moe": (_I, [_P, _P, _P, _P, _P, _P, _P, _L, _I, _I, _I, _I, _L, _L, _L, _L, _L, _P]),
    "gguf_b200_moe_a8_vec": (_I, [_P, _P, _P, _P, _L, _P, _L, _I, _I, _L, _L, _L, _L, _P]),
    "gguf_b200_mul_mat_vec_a8_noalloc": (_I, [_P, _P, _P, _I, _I, _L, _L, _L, _P]),
    "gguf_b200_mul_mat_vec_a8_tp": (_I, [_P, _P, _P, _P, _I, _I, _F, _I, _L, _P, _L, _I, _I, _L, _L, _I, _I, _P]),
    "gguf_b200_mul_mat_vec_a8_tp_rowpar": (_I, [_P, _P, _P, _P, _I, _I, _F, _I, _L, _P, _L, _I, _I, _L, _L, _I, _I, _P]),
    "gguf_b200_tp_unpack": (_I, [_P, _P, _I, _I, _L, _L, _P, _L, _I, _P]),
    "gguf_b200_tp_unpack_sum": (_I, [_P, _P, _I, _L, _L, _I, _P, _I, _P]),
    "gguf_b200_matmul_tp": (_I, [_I, _P, _P, _P, _P, _P, _I, _P, _L, _I, _I, _L, _L, _L, _I, _I, _P]),
    "gguf_b200_tp_wait": (_I, [_P, _P, _I, _I, _P]),
    "gguf_b200_set_wait_limit_cycles": (None, [_L]),
    "gguf_b200_noalloc_scratch_bytes": (_L, []),
    "gguf_b200_moe_block_size": (_I, [_I]),
    "gguf_b200_last_status": (_I, []),
    "gguf_b200_set_q4k_contract": (None, [_I]),
}


class GgufB200Error(RuntimeError):
    def __init__(self, code: int, op: str):
        self.code = code
        super().__init__(f"{op} failed ({code}): {lib().gguf_b200_error_string(code).decode()}")


def lib():
    """Load libgguf_b200.so (raises if it has not been built: there is no fallback)."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise ImportError(f"{_LIB_PATH} is not built; run gguf_b200/build.py")
        l = ctypes.CDLL(str(_LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            if hasattr(l, name):
                fn = getattr(l, name)
                fn.restype, fn.argtypes = res, args
        _lib = l
    return _lib


def _check(rc: int, op: str):
    if rc != 0:
        raise GgufB200Error(rc, op)


def _stream(t: torch.Tensor):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _ws(like: torch.Tensor, nbytes: int) -> torch.Tensor:
    return torch.empty(max(int(nbytes), 16), dtype=torch.uint8, device=like.device)


def k_of(W: torch.Tensor, qtype: int) -> int:
    return W.shape[-1] // lib().gguf_b200_type_size(qtype) * lib().gguf_b200_block_size(qtype)


def quantize_q8_1(X: torch.Tensor) -> torch.Tensor:
    M, K = X.shape
    out = torch.empty((M, lib().gguf_b200_q8_1_row_bytes(K)), dtype=torch.uint8, device=X.device)
    _check(lib().gguf_b200_quantize_q8_1(X.data_ptr(), _DT[X.dtype], out.data_ptr(), M, K, _stream(X)), "quantize_q8_1")
    return out


def dequantize(W: torch.Tensor, qtype: int, m: int, n: int, dtype=torch.float16) -> torch.Tensor:
    out = torch.empty((m, n), dtype=dtype, device=W.device)
    _check(lib().gguf_b200_dequantize(W.data_ptr(), qtype, out.data_ptr(), _DT[dtype], m * n, _stream(W)), "dequantize")
    return out


def dequantize_rows(W: torch.Tensor, row_ids: torch.Tensor, qtype: int, dtype=torch.float16) -> torch.Tensor:
    """[len(row_ids), K] = dequantized rows row_ids of the packed [rows, bytes] weight (embedding look-up)."""
    K = k_of(W, qtype)
    ids = row_ids.reshape(-1).to(torch.int64).contiguous()
    out = torch.empty((ids.numel(), K), dtype=dtype, device=W.device)
    _check(lib().gguf_b200_dequantize_rows(W.data_ptr(), qtype, ids.data_ptr(), ids.numel(), K, W.shape[0], out.data_ptr(),
                                           _DT[dtype], _stream(W)), "dequantize_rows")
    return out


def _matmul(fn_name: str, op: int, W: torch.Tensor, X: torch.Tensor, qtype: int, N: int) -> torch.Tensor:
    M, K = X.shape
    Y = torch.empty((M, N), dtype=X.dtype, device=X.device)
    nbytes = lib().gguf_b200_workspace_bytes(op, qtype, M, N, K)
    ws = _ws(X, nbytes)
    fn = getattr(lib(), fn_name)
    _check(fn(W.data_ptr(), X.data_ptr(), Y.data_ptr(), ws.data_ptr(), nbytes, qtype, _DT[X.dtype], M, N, K, _stream(X)), fn_name)
    return Y


def mul_mat_vec_a8(W, X, qtype, N):
    return _matmul("gguf_b200_mul_mat_vec_a8", OP_GEMV, W, X, qtype, N)


def gemv_prepare(X: torch.Tensor, qtype: int) -> torch.Tensor:
    """Quantize X once into a workspace that gemv_prepared() can reuse for several weights."""
    M, K = X.shape
    nbytes = lib().gguf_b200_workspace_bytes(OP_GEMV, qtype, M, 0, K)
    ws = _ws(X, nbytes)
    _check(lib().gguf_b200_gemv_prepare(X.data_ptr(), _DT[X.dtype], ws.data_ptr(), nbytes, qtype, M, K, _stream(X)),
           "gemv_prepare")
    return ws


def gemv_prepared(W, ws, qtype, M, N, K, dtype=torch.float16, out=None):
    Y = out if out is not None else torch.empty((M, N), dtype=dtype, device=W.device)
    _check(lib().gguf_b200_gemv_prepared(W.data_ptr(), ws.data_ptr(), Y.data_ptr(), qtype, _DT[dtype], M, N, K, _stream(W)),
           "gemv_prepared")
    return Y


def mul_mat_a8(W, X, qtype, N):
    return _matmul("gguf_b200_mul_mat_a8", OP_MMQ, W, X, qtype, N)


def dequant_matmul(W, X, qtype, N):
    return _matmul("gguf_b200_dequant_matmul", OP_DEQUANT_MATMUL, W, X, qtype, N)


def moe_a8(X, W, sorted_ids, expert_ids, n_post_pad, qtype, N, top_k, tokens):
    K = X.shape[1]
    Y = torch.empty((tokens * top_k, N), dtype=X.dtype, device=X.device)
    n_sorted = sorted_ids.numel()
    nbytes = lib().gguf_b200_workspace_bytes(OP_MOE, qtype, n_sorted, N, K)
    ws = _ws(X, nbytes)
    _check(lib().gguf_b200_moe_a8(X.data_ptr(), W.data_ptr(), Y.data_ptr(), ws.data_ptr(), nbytes, sorted_ids.data_ptr(),
                                  expert_ids.data_ptr(), n_post_pad.data_ptr(), n_sorted, W.stride(0), W.shape[0], qtype,
                                  _DT[X.dtype], tokens, top_k, N, K, _stream(X)), "moe_a8")
    return Y


ACT_SILU, ACT_GELU = 1, 2


def fused_moe(X, W13, W2, topk_ids, topk_weights, qtype13, qtype2, act=ACT_SILU):
    """The tiled MoE step in one call: X [T, H], W13 [E, 2I, bytes], W2 [E, H, bytes], topk_ids int32 [T, k],
    topk_weights float32 [T, k] -> [T, H]."""
    T, H = X.shape
    E, I2 = W13.shape[0], W13.shape[1]
    top_k = topk_ids.shape[1]
    I = I2 // 2
    Y = torch.empty((T, H), dtype=X.dtype, device=X.device)
    nbytes = lib().gguf_b200_fused_moe_workspace_bytes(qtype13, qtype2, _DT[X.dtype], T, top_k, E, H, I)
    ws = _ws(X, nbytes)
    ids = topk_ids.to(torch.int32).contiguous()
    tw = topk_weights.to(torch.float32).contiguous()
    _check(lib().gguf_b200_fused_moe(X.data_ptr(), W13.data_ptr(), W2.data_ptr(), Y.data_ptr(), ids.data_ptr(), tw.data_ptr(),
                                     ws.data_ptr(), nbytes, qtype13, qtype2, _DT[X.dtype], int(act), T, top_k, E, H, I,
                                     _stream(X)), "fused_moe")
    return Y


def moe_a8_vec(X, W, topk_ids, top_k, qtype, N, tokens):
    K = X.shape[1]
    Y = torch.empty((tokens * top_k, N), dtype=X.dtype, device=X.device)
    nbytes = lib().gguf_b200_workspace_bytes(OP_MOE_VEC, qtype, tokens, N, K)
    ws = _ws(X, nbytes)
    _check(lib().gguf_b200_moe_a8_vec(X.data_ptr(), W.data_ptr(), Y.data_ptr(), ws.data_ptr(), nbytes,
                                      topk_ids.data_ptr(), W.shape[0], qtype, _DT[X.dtype], tokens, top_k, N, K,
                                      _stream(X)), "moe_a8_vec")
    return Y


def mul_mat_vec_a8_noalloc(W, X, qtype, N):
    """GEMV through the entry point that takes no workspace (for hosts that cannot allocate one);
    only the output tensor is created here, by the caller's own allocator."""
    M, K = X.shape
    Y = torch.empty((M, N), dtype=X.dtype, device=X.device)
    _check(lib().gguf_b200_mul_mat_vec_a8_noalloc(W.data_ptr(), X.data_ptr(), Y.data_ptr(), qtype, _DT[X.dtype], M, N, K,
                                                  _stream(X)), "mul_mat_vec_a8_noalloc")
    return Y


def _ptr_array(ptrs):
    arr = (ctypes.c_void_p * len(ptrs))(*[int(p) for p in ptrs])
    return arr, ctypes.cast(arr, ctypes.c_void_p)


def mul_mat_vec_a8_tp(W_local, X, packet_ptrs, epochs_local, slot, slot_packets, qtype, rank, add_slot=-1,
                      add_scale=0.0, dtype=None, add_parts=1):
    """Rank `rank`'s rows of a decode GEMV, sent as tagged packets into every rank's packet arena
    (packet_ptrs: device addresses of the arenas, one per rank, mapped into this process).
    Activations x' = X + add_scale * v[add_slot] (X may be None when add_slot >= 0); v is a gathered
    vector (add_parts = 1) or the sum of the partial vectors of a row-parallel call (add_parts = world)."""
    world = len(packet_ptrs)
    n_local = W_local.shape[0]
    K = k_of(W_local, qtype)
    dt = X.dtype if X is not None else dtype
    nbytes = lib().gguf_b200_workspace_bytes(OP_GEMV, qtype, 1, n_local, K)
    ws = _ws(W_local, nbytes)
    keep, pa = _ptr_array(packet_ptrs)
    _check(lib().gguf_b200_mul_mat_vec_a8_tp(W_local.data_ptr(), X.data_ptr() if X is not None else None, pa,
                                             epochs_local.data_ptr(), int(slot), int(add_slot), float(add_scale),
                                             int(add_parts), int(slot_packets), ws.data_ptr(), nbytes, qtype, _DT[dt],
                                             n_local, K, int(rank), world, _stream(W_local)), "mul_mat_vec_a8_tp")


def mul_mat_vec_a8_tp_rowpar(W_local, X_local, packet_ptrs, epochs_local, slot, slot_packets, qtype, rank, add_slot=-1,
                             add_scale=0.0, dtype=None, add_parts=1):
    """Rank `rank`'s K-shard of a decode GEMV (W_local: every row's K_local columns; X_local: the
    rank's K_local activations): the fp32 partial sums go to every rank's packet arena; their sum
    (tp_unpack_sum, or the next call's add path with add_parts = world) is the all-reduced result."""
    world = len(packet_ptrs)
    n = W_local.shape[0]
    k_local = k_of(W_local, qtype)
    dt = X_local.dtype if X_local is not None else dtype
    nbytes = lib().gguf_b200_workspace_bytes(OP_GEMV, qtype, 1, n, k_local)
    ws = _ws(W_local, nbytes)
    keep, pa = _ptr_array(packet_ptrs)
    _check(lib().gguf_b200_mul_mat_vec_a8_tp_rowpar(W_local.data_ptr(), X_local.data_ptr() if X_local is not None else None, pa,
                                                    epochs_local.data_ptr(), int(slot), int(add_slot), float(add_scale),
                                                    int(add_parts), int(slot_packets), ws.data_ptr(), nbytes, qtype, _DT[dt],
                                                    n, k_local, int(rank), world, _stream(W_local)), "mul_mat_vec_a8_tp_rowpar")


def tp_unpack_sum(packets_local: torch.Tensor, epochs_local: torch.Tensor, slot: int, slot_packets: int, n: int, parts: int,
                  dtype=torch.float16, out=None) -> torch.Tensor:
    """The all-reduced vector of a row-parallel call: sum of the `parts` partial vectors of `slot`."""
    if out is None:
        out = torch.empty((n,), dtype=dtype, device=packets_local.device)
    _check(lib().gguf_b200_tp_unpack_sum(packets_local.data_ptr(), epochs_local.data_ptr(), int(slot), int(slot_packets), int(n),
                                         int(parts), out.data_ptr(), _DT[out.dtype], _stream(packets_local)), "tp_unpack_sum")
    return out


def tp_unpack(packets_local: torch.Tensor, epochs_local: torch.Tensor, slot0: int, nslots: int, slot_packets: int, n: int,
              dtype=torch.float16, out=None) -> torch.Tensor:
    """Plain [nslots, n] tensor of the gathered vectors of slots slot0 .. slot0+nslots-1."""
    if out is None:
        out = torch.empty((nslots, n), dtype=dtype, device=packets_local.device)
    _check(lib().gguf_b200_tp_unpack(packets_local.data_ptr(), epochs_local.data_ptr(), int(slot0), int(nslots),
                                     int(slot_packets), int(n), out.data_ptr(), out.stride(0), _DT[out.dtype],
                                     _stream(packets_local)), "tp_unpack")
    return out


def matmul_tp(op, W_local, X, y_ptrs, flag_ptrs, epochs_local, slot, qtype, rank):
    """Rank `rank`'s column block of a prefill GEMM (op = OP_MMQ or OP_DEQUANT_MATMUL), stored into
    every rank's gathered [M, world * N_local] output (y_ptrs); raises flag_ptrs[r][slot] on all ranks."""
    world = len(y_ptrs)
    M, K = X.shape
    n_local = W_local.shape[0]
    nbytes = lib().gguf_b200_workspace_bytes(op, qtype, M, n_local, K)
    ws = _ws(X, nbytes)
    k1, ya = _ptr_array(y_ptrs)
    k2, fa = _ptr_array(flag_ptrs)
    _check(lib().gguf_b200_matmul_tp(int(op), W_local.data_ptr(), X.data_ptr(), ya, fa, epochs_local.data_ptr(), int(slot),
                                     ws.data_ptr(), nbytes, qtype, _DT[X.dtype], M, n_local, K, int(rank), world,
                                     _stream(X)), "matmul_tp")


def tp_wait(flags_local: torch.Tensor, epochs_local: torch.Tensor, slot: int, world: int):
    _check(lib().gguf_b200_tp_wait(flags_local.data_ptr(), epochs_local.data_ptr(), int(slot), int(world),
                                   _stream(flags_local)), "tp_wait")


def set_wait_limit_cycles(cycles: int) -> None:
    lib().gguf_b200_set_wait_limit_cycles(int(cycles))


def last_status() -> int:
    return lib().gguf_b200_last_status()
