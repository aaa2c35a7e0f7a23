# SPDX-License-Identifier: Apache-2.0
"""Type sets that drive the dispatch of the GGUF matmul path (reference:
quantization/utils.py:46-75).  Plain GGML type ids; ``gguf.GGMLQuantizationType`` members are
IntEnums and compare equal to them."""
from __future__ import annotations

import logging

logger = logging.getLogger("vllm_gguf_plugin")

F32, F16, BF16 = 0, 1, 30
Q4_0, Q4_1, Q5_0, Q5_1, Q8_0, Q8_1 = 2, 3, 6, 7, 8, 9
Q2_K, Q3_K, Q4_K, Q5_K, Q6_K = 10, 11, 12, 13, 14
IQ2_XXS, IQ2_XS, IQ3_XXS, IQ1_S, IQ4_NL, IQ3_S, IQ2_S, IQ4_XS, IQ1_M = 16, 17, 18, 19, 20, 21, 22, 23, 29

UNQUANTIZED_TYPES = {F32, F16, BF16}
STANDARD_QUANT_TYPES = {Q4_0, Q4_1, Q5_0, Q5_1, Q8_0, Q8_1}
KQUANT_TYPES = {Q2_K, Q3_K, Q4_K, Q5_K, Q6_K}
IMATRIX_QUANT_TYPES = {IQ1_M, IQ1_S, IQ2_XXS, IQ2_XS, IQ2_S, IQ3_XXS, IQ3_S, IQ4_XS, IQ4_NL}
DEQUANT_TYPES = STANDARD_QUANT_TYPES | KQUANT_TYPES | IMATRIX_QUANT_TYPES
MMVQ_QUANT_TYPES = STANDARD_QUANT_TYPES | KQUANT_TYPES | IMATRIX_QUANT_TYPES
MMQ_QUANT_TYPES = STANDARD_QUANT_TYPES | KQUANT_TYPES

# block geometry of the types this build has kernels for: type -> (values, bytes) per block
SUPPORTED_QUANT_SIZES = {Q4_0: (32, 18), Q4_1: (32, 20), Q5_0: (32, 22), Q5_1: (32, 24), Q8_0: (32, 34),
                         Q2_K: (256, 84), Q3_K: (256, 110), Q4_K: (256, 144), Q5_K: (256, 176), Q6_K: (256, 210),
                         IQ2_XXS: (256, 66), IQ4_NL: (32, 18), IQ4_XS: (256, 136),
                         IQ2_XS: (256, 74), IQ2_S: (256, 82), IQ3_XXS: (256, 98), IQ3_S: (256, 110), IQ1_S: (256, 50),
                         IQ1_M: (256, 56)}   # (these six: decode GEMV; more tokens: dequantize + matmul, as in the reference)


def quant_sizes(weight_type: int) -> tuple[int, int]:
    """(values per block, bytes per block); gguf.GGML_QUANT_SIZES for the supported types."""
    try:
        return SUPPORTED_QUANT_SIZES[int(weight_type)]
    except KeyError:
        raise NotImplementedError(f"Unsupported GGUF quantization type: {int(weight_type)}") from None
