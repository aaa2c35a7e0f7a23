"""Host-side helpers of the B200 GGUF quantized-matmul library: build recipe, ctypes binding
of the C-ABI, synthetic block generators and the column-sharded tensor-parallel wrapper."""
