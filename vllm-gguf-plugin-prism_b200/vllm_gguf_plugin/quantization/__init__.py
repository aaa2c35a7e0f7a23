# SPDX-License-Identifier: Apache-2.0
"""Quantization methods of the GGUF matmul path (reference: vllm_gguf_plugin/quantization/)."""
from .fused_moe import GGUFMoEMethod, _fused_moe_gguf, fused_moe_gguf
from .linear import GGUFLinearMethod, _fused_mul_mat_gguf, fused_mul_mat_gguf

__all__ = ["GGUFLinearMethod", "GGUFMoEMethod", "fused_mul_mat_gguf", "fused_moe_gguf", "_fused_mul_mat_gguf",
           "_fused_moe_gguf"]
