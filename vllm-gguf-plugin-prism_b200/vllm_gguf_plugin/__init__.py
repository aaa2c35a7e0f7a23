"""Drop-in replacement for the GGUF quantized-matmul hot path of the vLLM GGUF plugin.

Same import names as the reference package for this path: ``vllm_gguf_plugin.ops`` (the six
operator entry points) and ``vllm_gguf_plugin.quantization`` (the linear / MoE methods and
their dispatchers).  Everything is backed by hand-written sm_100a kernels behind a C-ABI
(``libgguf_b200.so``); there is no Triton backend and no CPU fallback -- importing ``ops``
without the built extension raises.
"""

__all__ = ["ops"]
