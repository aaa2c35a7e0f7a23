// Test infrastructure only: exposes the reference plugin's internal q8_1
// activation quantizer (a static kernel of vllm_gguf_plugin/csrc/gguf/gguf_kernel.cu:32-85
// that no torch op returns) through a C symbol, so that GPU parity tests can
// compare bit patterns. This file contains no arithmetic of its own: it textually
// includes the reference translation unit from where it lies (REF_CSRC include path)
// and forwards to quantize_row_q8_1_cuda. Never linked into the product library.
#include "gguf/gguf_kernel.cu"

#include <cuda_bf16.h>

extern "C" int ref_quantize_q8_1(const void* x, int dtype /*0 f32, 1 f16, 2 bf16*/,
                                 void* out_blocks, int kx, int ky, void* stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case 0:
      quantize_row_q8_1_cuda<float>((const float*)x, out_blocks, kx, ky, s);
      break;
    case 1:
      quantize_row_q8_1_cuda<c10::Half>((const c10::Half*)x, out_blocks, kx, ky, s);
      break;
    case 2:
      quantize_row_q8_1_cuda<c10::BFloat16>((const c10::BFloat16*)x, out_blocks, kx, ky, s);
      break;
    default:
      return -1;
  }
  return (int)cudaGetLastError();
}
