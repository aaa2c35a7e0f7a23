# SPDX-License-Identifier: Apache-2.0
"""Operator facade of the GGUF quantized-matmul path (B200 build).

Mirrors the public functions of the reference's ``vllm_gguf_plugin/ops.py:181-286`` --
same names, argument order and meaning -- on top of the ``_C_gguf`` torch library built from
``csrc/`` (hand-written sm_100a kernels behind the C-ABI of ``include/gguf_b200.h``).

Differences from the reference, all deliberate:
* no Triton backend and no CPU fallback: if the extension is missing, import fails loudly;
  ``VLLM_GGUF_USE_CUDA`` is accepted for compatibility but selects nothing;
* supported block types are Q4_0, Q4_1, Q5_0, Q5_1, Q8_0, Q2_K, Q3_K, Q4_K, Q5_K, Q6_K (every type of the reference's
  tiled kernels, ggml_mul_mat_a8 / ggml_moe_a8), IQ2_XXS, IQ4_NL, IQ4_XS and, for ggml_dequantize, ggml_mul_mat_vec_a8
  and ggml_moe_a8_vec, IQ2_XS, IQ2_S, IQ3_XXS, IQ3_S, IQ1_S, IQ1_M -- with them every type of the reference's
  dequantize dispatch (dequantize.cuh:527-571) and of its GEMV dispatch is covered; any other type raises
  ``NotImplementedError`` (the reference silently returns zeros for an unknown type in its
  matmul switch, gguf_kernel.cu:236-289);
* ``ggml_moe_get_block_size`` returns this library's token-block size (64, tensor-core tile)
  instead of 4; callers already feed it to ``moe_align_block_size`` (fused_moe.py:64-68);
* ``ggml_dequantize_rows`` is new: the embedding look-up (index_select of rows + ggml_dequantize,
  quantization/vocal_embeds.py:88-96) as one kernel;
* ``ggml_fused_moe`` is new: the whole tiled MoE step of a layer in one call;
* ``ggml_dequant_matmul`` is new: the fused form of "ggml_dequantize then x @ W.T" that the
  reference uses for IQ types above the GEMV batch threshold (quantization/linear.py:50-54).
"""
from __future__ import annotations

import os

import torch

# GGML type ids (gguf.GGMLQuantizationType; the reference keeps them in triton/gemm/utils.py:5-24)
GGML_TYPE_Q4_0 = 2
GGML_TYPE_Q4_1 = 3
GGML_TYPE_Q5_0 = 6
GGML_TYPE_Q5_1 = 7
GGML_TYPE_Q8_0 = 8
GGML_TYPE_Q2_K = 10
GGML_TYPE_Q3_K = 11
GGML_TYPE_Q4_K = 12
GGML_TYPE_Q5_K = 13
GGML_TYPE_Q6_K = 14
GGML_TYPE_IQ2_XXS = 16
GGML_TYPE_IQ2_XS = 17
GGML_TYPE_IQ3_XXS = 18
GGML_TYPE_IQ1_S = 19
GGML_TYPE_IQ4_NL = 20
GGML_TYPE_IQ3_S = 21
GGML_TYPE_IQ2_S = 22
GGML_TYPE_IQ4_XS = 23
GGML_TYPE_IQ1_M = 29

# accepted for compatibility with the reference's switch (ops.py:39); there is one backend
_USE_CUDA = os.environ.get("VLLM_GGUF_USE_CUDA", "1") == "1"

try:
    from . import _C_gguf  # noqa: F401  (loading the module registers torch.ops._C_gguf.*)
except ImportError as exc:  # no silent fallback: the CUDA extension IS the product
    raise ImportError(
        "vllm_gguf_plugin._C_gguf (sm_100a kernels) is not built; run "
        "`python vllm-gguf-plugin-prism_b200/gguf_b200/build.py` from the repository root"
    ) from exc

_CUDA_AVAILABLE = True
_CUDA_ENABLED = True

# (values per block, bytes per block) -- gguf.GGML_QUANT_SIZES for the supported types
QUANT_SIZES = {
    GGML_TYPE_Q4_0: (32, 18),
    GGML_TYPE_Q4_1: (32, 20),
    GGML_TYPE_Q5_0: (32, 22),
    GGML_TYPE_Q5_1: (32, 24),
    GGML_TYPE_Q8_0: (32, 34),
    GGML_TYPE_Q4_K: (256, 144),
    GGML_TYPE_Q5_K: (256, 176),
    GGML_TYPE_Q6_K: (256, 210),
    GGML_TYPE_IQ2_XXS: (256, 66),
    GGML_TYPE_IQ4_NL: (32, 18),
    GGML_TYPE_IQ4_XS: (256, 136),
    # code-book types with a decode GEMV (and MoE GEMV) here; more tokens go through dequantize + matmul
    17: (256, 74),    # IQ2_XS
    22: (256, 82),    # IQ2_S
    18: (256, 98),    # IQ3_XXS
    21: (256, 110),   # IQ3_S
    19: (256, 50),    # IQ1_S
    29: (256, 56),    # IQ1_M
    GGML_TYPE_Q2_K: (256, 84),
    GGML_TYPE_Q3_K: (256, 110),
}
_CUDA_GEMV_QUANT_TYPES = frozenset(QUANT_SIZES)
# types that only ggml_dequantize serves (none at present: every type of the reference's dispatch has a GEMV too)
DEQUANT_ONLY_SIZES: dict = {}
_CUDA_DEQUANT_TYPES = _CUDA_GEMV_QUANT_TYPES | frozenset(DEQUANT_ONLY_SIZES)
_CUDA_GEMM_QUANT_TYPES = frozenset({GGML_TYPE_Q4_0, GGML_TYPE_Q4_1, GGML_TYPE_Q5_0, GGML_TYPE_Q5_1, GGML_TYPE_Q8_0,
                                    GGML_TYPE_Q2_K, GGML_TYPE_Q3_K, GGML_TYPE_Q4_K, GGML_TYPE_Q5_K, GGML_TYPE_Q6_K})
_DEQUANT_MATMUL_TYPES = frozenset({GGML_TYPE_IQ2_XXS, GGML_TYPE_IQ4_NL, GGML_TYPE_IQ4_XS})


def _require(quant_type: int, allowed, op: str) -> None:
    if int(quant_type) not in allowed:
        raise NotImplementedError(f"{op}: GGML type {int(quant_type)} has no sm_100a kernel in this build "
                                  f"(supported: {sorted(allowed)})")


# --- fake (meta) implementations, needed under torch.compile (reference: ops.py:110-175) ---

try:
    from torch.library import register_fake
except ImportError:  # older torch
    from torch.library import impl_abstract as register_fake


@register_fake("_C_gguf::ggml_dequantize")
def _ggml_dequantize_fake(W, quant_type, m, n, dtype=None):
    return torch.empty((m, n), dtype=dtype or torch.float16, device=W.device)


@register_fake("_C_gguf::ggml_mul_mat_vec_a8")
def _ggml_mul_mat_vec_a8_fake(W, X, quant_type, row):
    return torch.empty((X.shape[0], row), dtype=X.dtype, device=W.device)


@register_fake("_C_gguf::ggml_mul_mat_a8")
def _ggml_mul_mat_a8_fake(W, X, quant_type, row):
    return torch.empty((X.size(0), row), dtype=X.dtype, device=W.device)


@register_fake("_C_gguf::dequant_matmul")
def _dequant_matmul_fake(W, X, quant_type, row):
    return torch.empty((X.size(0), row), dtype=X.dtype, device=W.device)


@register_fake("_C_gguf::dequantize_rows")
def _dequantize_rows_fake(W, ids, quant_type, dtype=None):
    block, size = (QUANT_SIZES | DEQUANT_ONLY_SIZES)[int(quant_type)]
    return torch.empty((ids.shape[0], W.shape[1] // size * block), dtype=dtype or torch.float16, device=W.device)


@register_fake("_C_gguf::fused_moe")
def _fused_moe_fake(X, W13, W2, topk_weights, topk_ids, type13, type2, act):
    return torch.empty_like(X)


@register_fake("_C_gguf::ggml_moe_a8")
def _ggml_moe_a8_fake(X, W, sorted_token_ids, expert_ids, num_tokens_post_padded, quant_type, row, top_k, tokens):
    return torch.empty((X.size(0) * top_k, row), dtype=X.dtype, device=W.device)


@register_fake("_C_gguf::ggml_moe_a8_vec")
def _ggml_moe_a8_vec_fake(X, W, topk_ids, top_k, quant_type, row, tokens):
    return torch.empty((X.size(0) * top_k, row), dtype=X.dtype, device=W.device)


# --- public API (reference: ops.py:181-286) ---


def ggml_dequantize(W: torch.Tensor, quant_type: int, m: int, n: int, dtype: torch.dtype | None) -> torch.Tensor:
    _require(quant_type, _CUDA_DEQUANT_TYPES, "ggml_dequantize")
    return torch.ops._C_gguf.ggml_dequantize(W, quant_type, m, n, dtype)


def ggml_mul_mat_vec_a8(W: torch.Tensor, X: torch.Tensor, quant_type: int, row: int) -> torch.Tensor:
    _require(quant_type, _CUDA_GEMV_QUANT_TYPES, "ggml_mul_mat_vec_a8")
    return torch.ops._C_gguf.ggml_mul_mat_vec_a8(W, X, quant_type, row)


def ggml_mul_mat_a8(W: torch.Tensor, X: torch.Tensor, quant_type: int, row: int) -> torch.Tensor:
    _require(quant_type, _CUDA_GEMM_QUANT_TYPES, "ggml_mul_mat_a8")
    return torch.ops._C_gguf.ggml_mul_mat_a8(W, X, quant_type, row)


def ggml_dequant_matmul(W: torch.Tensor, X: torch.Tensor, quant_type: int, row: int) -> torch.Tensor:
    """x @ dequantize(W).T in one kernel, unquantized fp16/bf16 activations (IQ2_XXS, IQ4_XS)."""
    _require(quant_type, _DEQUANT_MATMUL_TYPES, "ggml_dequant_matmul")
    return torch.ops._C_gguf.dequant_matmul(W, X, quant_type, row)


def ggml_dequantize_rows(W: torch.Tensor, ids: torch.Tensor, quant_type: int, dtype: torch.dtype | None) -> torch.Tensor:
    """Rows ``ids`` (1-D int64) of the packed ``[rows, bytes]`` weight, dequantized to ``[len(ids), K]``:
    the embedding look-up in one kernel (the reference does index_select, then ggml_dequantize)."""
    _require(quant_type, _CUDA_DEQUANT_TYPES, "ggml_dequantize_rows")
    return torch.ops._C_gguf.dequantize_rows(W, ids, quant_type, dtype)


def ggml_moe_a8(
    X: torch.Tensor,
    W: torch.Tensor,
    sorted_token_ids: torch.Tensor,
    expert_ids: torch.Tensor,
    num_tokens_post_padded: torch.Tensor,
    quant_type: int,
    row: int,
    top_k: int,
    tokens: int,
) -> torch.Tensor:
    _require(quant_type, _CUDA_GEMM_QUANT_TYPES, "ggml_moe_a8")
    return torch.ops._C_gguf.ggml_moe_a8(
        X, W, sorted_token_ids, expert_ids, num_tokens_post_padded, quant_type, row, top_k, tokens
    )


MOE_ACTIVATIONS = {"silu": 1, "gelu": 2}


def ggml_fused_moe(X: torch.Tensor, W13: torch.Tensor, W2: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor,
                   quant_type: int, quant_type2: int, activation: str) -> torch.Tensor:
    """The tiled MoE step of one layer in one call: alignment, gate/up expert GEMM, activation, down
    expert GEMM, routing weights and the top-k sum (the reference runs six ops for it,
    quantization/fused_moe.py:56-95).  X [T, H] -> [T, H]."""
    _require(quant_type, _CUDA_GEMM_QUANT_TYPES, "ggml_fused_moe")
    _require(quant_type2, _CUDA_GEMM_QUANT_TYPES, "ggml_fused_moe")
    return torch.ops._C_gguf.fused_moe(X, W13, W2, topk_weights.to(torch.float32).contiguous(),
                                       topk_ids.to(torch.int32).contiguous(), quant_type, quant_type2,
                                       MOE_ACTIVATIONS[activation])


def ggml_moe_a8_vec(
    X: torch.Tensor,
    W: torch.Tensor,
    topk_ids: torch.Tensor,
    top_k: int,
    quant_type: int,
    row: int,
    tokens: int,
) -> torch.Tensor:
    _require(quant_type, _CUDA_GEMV_QUANT_TYPES, "ggml_moe_a8_vec")
    return torch.ops._C_gguf.ggml_moe_a8_vec(X, W, topk_ids, top_k, quant_type, row, tokens)


def ggml_moe_get_block_size(quant_type: int) -> int:
    _require(quant_type, _CUDA_GEMM_QUANT_TYPES, "ggml_moe_get_block_size")
    return torch.ops._C_gguf.ggml_moe_get_block_size(quant_type)


def moe_sum(input: torch.Tensor, output: torch.Tensor) -> None:
    """Sum over the top-k axis: [tokens, top_k, hidden] -> [tokens, hidden] (reference ops.py:285-286
    forwards to vLLM's ``_moe_C.moe_sum``; without vLLM's extension the same reduction is torch.sum)."""
    moe_c = getattr(torch.ops, "_moe_C", None)
    if moe_c is not None and hasattr(moe_c, "moe_sum"):
        moe_c.moe_sum(input, output)
    else:
        torch.sum(input, dim=1, out=output)
