// The small kernels that turn the MoE step around the two expert GEMMs into one call
// (reference: _fused_moe_gguf, quantization/fused_moe.py:56-95 -- there the alignment, the
// activation, the routing-weight multiply and the top-k sum are four separate library ops with
// their own launches and two [tokens*top_k, .] round trips through memory):
//
//   moe_align_*        expert-sorted, block-padded slot lists (what vLLM's moe_align_block_size
//                      gives the reference, fused_moe.py:66-68): slot s = token*top_k + j goes to
//                      the list of expert topk_ids[s]; every expert's list is padded to a multiple
//                      of the token-block size with the sentinel `slots`; one expert id per block.
//                      Slots keep their order inside an expert (stable), so the result is unique.
//   moe_sum_kernel     out[t] = sum over j of y[t*top_k + j]   (fp32 accumulation, one rounding)
//
// The activation (silu/gelu(gate) * up) runs inside the activation quantizer of the second GEMM
// (quantize_q8_1.cu, act mode) and the routing weights inside that GEMM's epilogue (mmq.cu), so
// neither the activated matrix nor the weighted one exists in memory.
#include "common.cuh"
#include "kernels.h"

namespace gguf_b200 {

// one warp per expert: how many slots chose it
__global__ void __launch_bounds__(256) moe_align_count_kernel(const int32_t* __restrict__ topk_ids, int64_t slots, int n_experts,
                                                              int32_t* __restrict__ counts) {
  pdl_trigger();
  pdl_wait();
  const int e = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (e >= n_experts) return;
  int c = 0;
  for (int64_t s = lane; s < slots; s += 32) c += topk_ids[s] == e ? 1 : 0;
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) c += __shfl_xor_sync(0xffffffffu, c, m);
  if (lane == 0) counts[e] = c;
}

// one CTA: padded prefix over the experts -> starts[e], the total, expert_ids per block, and the
// sentinel in every position (the placing kernel then overwrites the real ones)
__global__ void __launch_bounds__(1024) moe_align_offsets_kernel(const int32_t* __restrict__ counts, int n_experts, int block,
                                                                 int64_t slots, int64_t n_sorted, int32_t* __restrict__ starts,
                                                                 int32_t* __restrict__ sorted_ids, int32_t* __restrict__ expert_ids,
                                                                 int32_t* __restrict__ n_post_pad) {
  pdl_trigger();
  pdl_wait();
  __shared__ int32_t s_start[257];
  if (threadIdx.x == 0) {
    int32_t pos = 0;
    for (int e = 0; e < n_experts; ++e) {
      s_start[e] = pos;
      pos += (counts[e] + block - 1) / block * block;
    }
    s_start[n_experts] = pos;
    n_post_pad[0] = pos;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) starts[e] = s_start[e];
  for (int64_t i = threadIdx.x; i < n_sorted; i += blockDim.x) sorted_ids[i] = (int32_t)slots;
  const int64_t nblocks = n_sorted / block;
  for (int64_t b = threadIdx.x; b < nblocks; b += blockDim.x) {
    const int32_t pos = (int32_t)(b * block);
    int e = 0;   // the expert whose padded range holds this block (blocks past the total keep expert 0: never used)
    for (int k = 0; k < n_experts; ++k)
      if (pos >= s_start[k] && pos < s_start[k + 1]) e = k;
    expert_ids[b] = e;
  }
}

// one warp per expert: its slots, in slot order, to positions starts[e], starts[e] + 1, ...
__global__ void __launch_bounds__(256) moe_align_place_kernel(const int32_t* __restrict__ topk_ids, int64_t slots, int n_experts,
                                                              const int32_t* __restrict__ starts, int32_t* __restrict__ sorted_ids) {
  pdl_trigger();
  pdl_wait();
  const int e = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (e >= n_experts) return;
  int32_t pos = starts[e];
  for (int64_t s0 = 0; s0 < slots; s0 += 32) {
    const int64_t s = s0 + lane;
    const bool mine = s < slots && topk_ids[s] == e;
    const unsigned m = __ballot_sync(0xffffffffu, mine);
    if (mine) sorted_ids[pos + __popc(m & ((1u << lane) - 1u))] = (int32_t)s;
    pos += __popc(m);
  }
}

int64_t moe_align_sorted_len(int64_t slots, int n_experts, int block) {
  const int64_t worst = slots + (int64_t)n_experts * (block - 1);
  return (worst + block - 1) / block * block;
}

// scratch: counts[E] | starts[E]  (int32)
int launch_moe_align(const int32_t* topk_ids, int64_t slots, int n_experts, int block, int32_t* scratch, int32_t* sorted_ids,
                     int32_t* expert_ids, int32_t* n_post_pad, cudaStream_t stream) {
  if (n_experts < 1 || n_experts > 256 || block < 1) return E_BAD_SHAPE;
  const int64_t n_sorted = moe_align_sorted_len(slots, n_experts, block);
  int32_t* counts = scratch;
  int32_t* starts = scratch + n_experts;
  const unsigned ge = (unsigned)((n_experts + 7) / 8);
  if (launch_pdl(moe_align_count_kernel, dim3(ge), dim3(256), 0, stream, topk_ids, slots, n_experts, counts) != cudaSuccess) return E_CUDA;
  if (launch_pdl(moe_align_offsets_kernel, dim3(1), dim3(1024), 0, stream, (const int32_t*)counts, n_experts, block, slots, n_sorted,
                 starts, sorted_ids, expert_ids, n_post_pad) != cudaSuccess)
    return E_CUDA;
  if (launch_pdl(moe_align_place_kernel, dim3(ge), dim3(256), 0, stream, topk_ids, slots, n_experts, (const int32_t*)starts, sorted_ids) !=
      cudaSuccess)
    return E_CUDA;
  return E_OK;
}

template <typename T>
__global__ void __launch_bounds__(256) moe_sum_kernel(const T* __restrict__ y, T* __restrict__ out, const int32_t* __restrict__ topk_ids,
                                                      int n_experts, int64_t tokens, int top_k, int64_t h) {
  pdl_trigger();
  pdl_wait();
  const int64_t total = tokens * h;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = i / h, c = i - t * h;
    float s = 0.f;
    for (int j = 0; j < top_k; ++j) {
      const int e = topk_ids[t * top_k + j];
      if (e >= 0 && e < n_experts) s += to_float<T>(y[(t * top_k + j) * h + c]);   // a slot without a valid expert contributes nothing
    }
    out[i] = from_float<T>(s);
  }
}

int launch_moe_sum(const void* y, void* out, const int32_t* topk_ids, int n_experts, int64_t tokens, int64_t top_k, int64_t h,
                   int dtype, cudaStream_t stream) {
  const int64_t total = tokens * h;
  if (total == 0) return E_OK;
  const unsigned grid = (unsigned)((total + 255) / 256 > 148 * 8 ? 148 * 8 : (total + 255) / 256);
  cudaError_t e;
  switch (dtype) {
    case DT_F32:
      e = launch_pdl(moe_sum_kernel<float>, dim3(grid), dim3(256), 0, stream, (const float*)y, (float*)out, topk_ids, n_experts, tokens, (int)top_k, h);
      break;
    case DT_F16:
      e = launch_pdl(moe_sum_kernel<__half>, dim3(grid), dim3(256), 0, stream, (const __half*)y, (__half*)out, topk_ids, n_experts, tokens, (int)top_k, h);
      break;
    case DT_BF16:
      e = launch_pdl(moe_sum_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, stream, (const __nv_bfloat16*)y, (__nv_bfloat16*)out, topk_ids, n_experts, tokens, (int)top_k, h);
      break;
    default:
      return E_BAD_DTYPE;
  }
  return e == cudaSuccess ? E_OK : E_CUDA;
}

}  // namespace gguf_b200
