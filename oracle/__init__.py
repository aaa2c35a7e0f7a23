"""CPU oracle of the GGUF quantized-matmul path -- test infrastructure, never a product path.

Only tests/, the smoke check and the CPU-baseline / reference arms of the benchmark may
import this package.  ``oracle.cpu`` wraps the C restatement (gguf_oracle.c);
``oracle.build_ref`` builds the reference plugin's own CUDA extension for GPU parity runs.
"""
