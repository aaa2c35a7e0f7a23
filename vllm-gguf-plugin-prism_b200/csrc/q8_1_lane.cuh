// One lane's share of the q8_1 quantization of a block of 32 values (lane j = value j).
// Shared by the standalone quantizer (quantize_q8_1.cu) and the decode GEMV that quantizes its
// activations itself (gemv1.cu).  Both translation units are compiled with --use_fast_math, like
// the reference (setup.py:34-42), so the two fp32 divisions below are the same approximate
// instructions everywhere -- the codes are bit-identical to the reference's quantize_q8_1
// (gguf_kernel.cu:32-69) whichever kernel produces them.
#pragma once

#include "common.cuh"

namespace gguf_b200 {

struct Q8Lane {
  float d;     // fp32 scale before fp16 rounding (the quantity q was divided by)
  float sum;   // fp32 butterfly sum of the 32 inputs
  int q;       // this lane's int8 code
};

__device__ __forceinline__ Q8Lane quantize_lane(float xi) {
  float amax = fabsf(xi);
  float sum = xi;
#pragma unroll
  for (int mask = 16; mask > 0; mask >>= 1) {
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, mask, 32));
    sum += __shfl_xor_sync(0xffffffffu, sum, mask, 32);
  }
  Q8Lane r;
  r.d = amax / 127;
  const int8_t q = amax == 0.0f ? 0 : roundf(xi / r.d);
  r.q = q;
  r.sum = sum;
  return r;
}

// gather the four int8 codes of lanes 4i..4i+3 into one word held by lane 4i
__device__ __forceinline__ uint32_t pack4(int q, int lane) {
  uint32_t b = (uint32_t)q & 0xffu;
  uint32_t b1 = __shfl_down_sync(0xffffffffu, b, 1);
  uint32_t b2 = __shfl_down_sync(0xffffffffu, b, 2);
  uint32_t b3 = __shfl_down_sync(0xffffffffu, b, 3);
  (void)lane;
  return b | (b1 << 8) | (b2 << 16) | (b3 << 24);
}

}  // namespace gguf_b200
