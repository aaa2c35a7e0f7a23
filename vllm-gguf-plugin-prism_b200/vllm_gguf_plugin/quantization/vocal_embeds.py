# SPDX-License-Identifier: Apache-2.0
"""Embedding caller of the dequantize kernel (reference: quantization/vocal_embeds.py:79-98).

``_apply_gguf_embedding`` keeps the reference's signature.  Where the reference copies the
selected rows with ``index_select`` and dequantizes the copy, this build gathers inside the
dequantize kernel (``ops.ggml_dequantize_rows``); hidden sizes that are not a multiple of 256 take
the reference's two steps.  The vLLM embedding *method* class (weight creation and loading) is
outside this path."""
from __future__ import annotations

import torch

from .. import ops
from .utils import DEQUANT_TYPES, UNQUANTIZED_TYPES, quant_sizes


def _apply_gguf_embedding(x: torch.Tensor, weight: torch.Tensor, weight_type: int, hidden_size: int,
                          dtype: torch.dtype | None = None) -> torch.Tensor:
    if weight_type in UNQUANTIZED_TYPES:
        return torch.embedding(weight, x)
    if weight_type in DEQUANT_TYPES:
        block_size, type_size = quant_sizes(weight_type)
        x_flat = x.flatten()
        assert hidden_size == weight.shape[1] // type_size * block_size
        if hidden_size % 256 == 0:
            dequant = ops.ggml_dequantize_rows(weight, x_flat.to(torch.int64).contiguous(), weight_type, dtype)
        else:
            quant = torch.index_select(weight, dim=0, index=x_flat)
            dequant = ops.ggml_dequantize(quant, weight_type, hidden_size, x_flat.shape[0], dtype)
        return dequant.view(*x.shape, hidden_size)
    raise NotImplementedError(f"Unsupported GGUF quantization type: {int(weight_type)}")


def _apply_gguf_embedding_fake(x: torch.Tensor, weight: torch.Tensor, weight_type: int, hidden_size: int,
                               dtype: torch.dtype | None = None) -> torch.Tensor:
    return torch.empty(*x.shape, hidden_size, dtype=dtype, device=x.device)
