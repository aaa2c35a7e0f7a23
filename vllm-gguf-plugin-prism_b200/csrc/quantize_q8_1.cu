// q8_1 activation quantization: every matmul entry point of the path first turns the
// fp32/fp16/bf16 activations into blocks of 32 int8 values with an fp16 scale d = amax/127
// and the fp16 sum of the unquantized inputs (reference: quantize_q8_1,
// vllm_gguf_plugin/csrc/gguf/gguf_kernel.cu:32-69; launcher :71-85, K padded with zeros to a
// multiple of 512).
//
// The values must equal the reference's bit for bit.  Two things make that so:
//  * lane j of a warp holds element j of a block and the amax/sum reductions use the same
//    xor-butterfly (masks 16,8,4,2,1), so the fp32 sum is accumulated in the same order;
//  * this translation unit is compiled with --use_fast_math like the reference
//    (setup.py:34-42), and d and q use the same expression forms (amax / 127, roundf(x / d)),
//    so the approximate fp32 divisions are the same instructions.
//
// Three output layouts share one device routine:
//   REF  : the 36-byte block_q8_1 records (what gguf_b200_quantize_q8_1 returns)
//   SOA  : int8 qs[M][Kpad] followed by float2 ds[M][Kpad/32] -- the layout the GEMV kernels
//          stage into shared memory with 16-byte copies.  ds.x = d (fp16 value as float);
//          ds.y = the fp16 sum as float, or, for the Q4_K GEMV, d * sum(q) because that
//          kernel's min term uses the quantized sum (vecdotq.cuh:342-345).
//   F16  : x^[m][k] = half(d * q) in a K-major matrix [Mpad][ldb] for the tensor-core kernels,
//          plus per-block correction columns appended after K (see mmq.cu).
#include "common.cuh"
#include "kernels.h"
#include "q8_1_lane.cuh"

namespace gguf_b200 {

template <typename in_t, int MODE>
__global__ void __launch_bounds__(256) quantize_q8_1_kernel(const in_t* __restrict__ x, uint8_t* __restrict__ out,
                                                            int64_t M, int64_t K, int64_t kpad, int sum_mode,
                                                            int64_t ldb, int corr_mode, const int32_t* __restrict__ gather_ids,
                                                            int64_t gather_div, int64_t gather_limit, Q8Tp tp) {
  pdl_trigger();  // the consumer kernel may start its weight prefetch now; it waits for this grid before reading
  pdl_wait();     // the activations (and the scratch we overwrite) belong to earlier kernels
  // tensor-parallel decode: this launch's number for the GEMV behind it, and the tag of the
  // gathered vector (written by all ranks' GEMV kernels into this rank's memory) that is added to x
  if (MODE == Q8_MODE_SOA && tp.bump && blockIdx.x == 0 && threadIdx.x == 0) *tp.bump += 1u;
  const unsigned add_tag = (MODE == Q8_MODE_SOA && tp.add) ? *tp.add_epoch : 0u;
  const int lane = threadIdx.x & 31;
  const int64_t nbr = kpad / 32;                                   // blocks per row
  const int64_t total = M * nbr;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  for (int64_t b = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); b < total; b += warps) {
    const int64_t row = b / nbr, kb = b - row * nbr;
    const int64_t k = kb * 32 + lane;
    // F16 mode may gather: output row `row` takes input row gather_ids[row] / gather_div
    // (MoE: sorted slot -> token); ids at or beyond gather_limit are padding and give a zero row.
    int64_t src = row;
    bool have = true;
    if (MODE == Q8_MODE_F16 && gather_ids) {
      const int64_t id = gather_ids[row];
      have = id >= 0 && id < gather_limit;
      src = have ? id / gather_div : 0;
    }
    float xi = (x && have && k < K) ? to_float<in_t>(x[src * K + k]) : 0.0f;
    if (MODE == Q8_MODE_SOA && tp.add && k < K) {   // (one vector: row == 0)
      float a;
      if (tp.add_parts > 1) {   // all-reduce of a row-parallel call: partial vectors in fp32, summed in rank order, rounded once
        a = 0.f;
        for (int r = 0; r < tp.add_parts; ++r) {
          float part;
          if (!packet_read<float>(tp.add, r * tp.add_stride + k, add_tag, tp.limit_cycles, part)) atomicExch(tp.status, E_TIMEOUT);
          a += part;
        }
        a = to_float<in_t>(from_float<in_t>(a));
      } else if (!packet_read<in_t>(tp.add, k, add_tag, tp.limit_cycles, a)) {
        atomicExch(tp.status, E_TIMEOUT);
      }
      xi = to_float<in_t>(from_float<in_t>(xi + tp.add_scale * a));   // x' is a vector of the activation type
    }
    const Q8Lane r = quantize_lane(xi);
    const __half hd = __float2half(r.d), hs = __float2half(r.sum);
    if (MODE == Q8_MODE_REF) {
      uint8_t* blk = out + b * 36;
      blk[4 + lane] = (uint8_t)r.q;
      if (lane == 0) {
        *reinterpret_cast<__half*>(blk) = hd;
        *reinterpret_cast<__half*>(blk + 2) = hs;
      }
    } else if (MODE == Q8_MODE_SOA) {
      const uint32_t w = pack4(r.q, lane);
      if ((lane & 3) == 0) *reinterpret_cast<uint32_t*>(out + row * kpad + kb * 32 + lane) = w;
      int qs = r.q;
#pragma unroll
      for (int mask = 16; mask > 0; mask >>= 1) qs += __shfl_xor_sync(0xffffffffu, qs, mask);
      if (lane == 0) {
        const float d8 = __half2float(hd);
        float2 ds;
        ds.x = d8;
        ds.y = sum_mode ? d8 * (float)qs : __half2float(hs);
        reinterpret_cast<float2*>(out + M * kpad)[b] = ds;
      }
    } else {  // Q8_MODE_F16: B operand of the tensor-core kernels
      __half* xb = reinterpret_cast<__half*>(out);
      const float d8 = __half2float(hd);
      xb[row * ldb + k] = __float2half_rn(d8 * (float)r.q);
      if (corr_mode != CORR_NONE) {
        int qs = r.q;
#pragma unroll
        for (int mask = 16; mask > 0; mask >>= 1) qs += __shfl_xor_sync(0xffffffffu, qs, mask);
        if (lane == 0) {
          // the reference's tiled kernels subtract (weight offset) * s8, with s8 the fp16 sum of
          // the unquantized inputs (vecdotq.cuh:61-64, :369-372).  The tensor-core product already
          // contains (offset-free part) . x^; the appended column carries what is left.
          const float s8 = __half2float(hs);
          float c;
          if (corr_mode == CORR_Q4_0) c = -8.0f * s8;                    // weights decoded as q * d: the format's -8 * d meets the sum here
          else c = corr_mode == CORR_PLUS ? s8 : -s8;                    // CORR_PLUS: + m * s8;  CORR_MIN: minus min * s8
          xb[row * ldb + kpad + kb] = __float2half_rn(c);
        }
        // zero the tail of the correction area so that padded contraction columns contribute nothing
        if (kb == 0)
          for (int64_t c = kpad + nbr + lane; c < ldb; c += 32) xb[row * ldb + c] = __float2half_rn(0.f);
      }
    }
  }
}


// F16 layout, eight inputs per thread (16-byte loads and stores): four lanes own one block of 32.
// The reference's butterfly adds element i to element i^16, then i^8, i^4, i^2, i^1; with lane
// t of a quad holding elements 8t..8t+7 the first two levels are shuffles across the quad (lane
// ^2, lane ^1) and the last three are adds inside the thread, in the same order, so the fp32 sum
// has the same bits.  perm = 1 stores every group of four values in the order (0,2,1,3) (see
// Stage64 in mmq_decode.cuh).
// act != 0 (fused MoE step): the input rows are [gate | up] of x_ld = 2K values and the value that
// is quantized is act(gate) * up, formed as the reference's separate activation op forms it --
// silu(g) = g / (1 + exp(-g)) (gelu: 0.5 g (1 + erf(g / sqrt 2))) rounded to the activation type,
// then multiplied by up in that type (one more rounding) -- so the activated matrix never exists
// in memory.  (This file is built with fast-math: exp() is the hardware approximation, which can
// move the rounded silu by one unit in the last place in rare cases.)
template <typename in_t> __device__ __forceinline__ float act_mul(int act, float g, float u) {
  const float a = act == 1 ? g / (1.0f + expf(-g)) : 0.5f * g * (1.0f + erff(g * 0.70710678118654752f));
  return to_float<in_t>(from_float<in_t>(to_float<in_t>(from_float<in_t>(a)) * u));
}

template <typename in_t>
__global__ void __launch_bounds__(256) quantize_f16x8_kernel(const in_t* __restrict__ x, __half* __restrict__ xb, int64_t M, int64_t K,
                                                             int64_t kpad, int64_t ldb, int corr_mode, int perm,
                                                             const int32_t* __restrict__ gather_ids, int64_t gather_div,
                                                             int64_t gather_limit, int act, int64_t x_ld) {
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31, t = lane & 3;
  const int64_t nbr = kpad / 32;                                   // blocks per row
  const int64_t total = M * nbr;                                   // blocks in all
  const int64_t stride = (int64_t)gridDim.x * (blockDim.x >> 2);
  // every lane of a warp runs the same number of iterations (the shuffles need all of them)
  const int64_t first = (int64_t)blockIdx.x * (blockDim.x >> 2) + (threadIdx.x >> 5) * 8;
  for (int64_t b0 = first; b0 < total; b0 += stride) {
    const int64_t b = b0 + (lane >> 2);
    const bool inb = b < total;
    const int64_t row = inb ? b / nbr : 0, kb = inb ? b - row * nbr : 0;
    const int64_t k = kb * 32 + 8 * t;
    int64_t src = row;
    bool have = inb;
    if (gather_ids && inb) {
      const int64_t id = gather_ids[row];
      have = id >= 0 && id < gather_limit;
      src = have ? id / gather_div : 0;
    }
    float v[8];
    if (act) {
      if (have && k + 8 <= K && sizeof(in_t) == 2 && K % 8 == 0 && x_ld % 8 == 0) {
        const uint4 ga = *reinterpret_cast<const uint4*>(x + src * x_ld + k), ua = *reinterpret_cast<const uint4*>(x + src * x_ld + K + k);
        const in_t* ge = reinterpret_cast<const in_t*>(&ga);
        const in_t* ue = reinterpret_cast<const in_t*>(&ua);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = act_mul<in_t>(act, to_float<in_t>(ge[j]), to_float<in_t>(ue[j]));
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          v[j] = (have && k + j < K) ? act_mul<in_t>(act, to_float<in_t>(x[src * x_ld + k + j]), to_float<in_t>(x[src * x_ld + K + k + j])) : 0.0f;
      }
    } else if (have && k + 8 <= K) {
      if (sizeof(in_t) == 4) {
        const float4 a = *reinterpret_cast<const float4*>(x + src * K + k), c = *reinterpret_cast<const float4*>(x + src * K + k + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = c.x; v[5] = c.y; v[6] = c.z; v[7] = c.w;
      } else {
        const uint4 a = *reinterpret_cast<const uint4*>(x + src * K + k);
        const in_t* e = reinterpret_cast<const in_t*>(&a);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = to_float<in_t>(e[j]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = (have && k + j < K) ? to_float<in_t>(x[src * K + k + j]) : 0.0f;
    }
    float amax = 0.f, sm[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      amax = fmaxf(amax, fabsf(v[j]));
      sm[j] = v[j] + __shfl_xor_sync(0xffffffffu, v[j], 2, 32);          // i ^ 16
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) sm[j] += __shfl_xor_sync(0xffffffffu, sm[j], 1, 32);   // i ^ 8
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2, 32));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1, 32));
    float s4[4], s2[2];
#pragma unroll
    for (int j = 0; j < 4; ++j) s4[j] = sm[j] + sm[j + 4];               // i ^ 4
#pragma unroll
    for (int j = 0; j < 2; ++j) s2[j] = s4[j] + s4[j + 2];               // i ^ 2
    const float sum = s2[0] + s2[1];                                      // i ^ 1
    const float d = amax / 127;
    const __half hd = __float2half(d), hs = __float2half(sum);
    const float d8 = __half2float(hd);
    int q[8], qs = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int8_t qq = amax == 0.0f ? 0 : roundf(v[j] / d);
      q[j] = qq;
      qs += q[j];
    }
    if (inb) {
      __half o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int jj = perm ? ((j & 4) | ((j & 1) << 1) | ((j >> 1) & 1)) : j;   // position jj holds value j
        o[jj] = __float2half_rn(d8 * (float)q[j]);
      }
      *reinterpret_cast<uint4*>(xb + row * ldb + k) = *reinterpret_cast<const uint4*>(o);
    }
    if (corr_mode != CORR_NONE) {
      qs += __shfl_xor_sync(0xffffffffu, qs, 2, 32);
      qs += __shfl_xor_sync(0xffffffffu, qs, 1, 32);
      if (inb && t == 0) {
        const float s8 = __half2float(hs);
        const float c = corr_mode == CORR_Q4_0 ? -8.0f * s8 : (corr_mode == CORR_PLUS ? s8 : -s8);   // see quantize_q8_1_kernel
        xb[row * ldb + kpad + kb] = __float2half_rn(c);
      }
      if (inb && kb == 0)
        for (int64_t c = kpad + nbr + t; c < ldb; c += 4) xb[row * ldb + c] = __float2half_rn(0.f);
    }
  }
}

template <int MODE>
static int launch_mode(const void* x, int x_dtype, void* out, int64_t M, int64_t K, int sum_mode, int64_t ldb,
                       int corr_mode, const int32_t* gid, int64_t gdiv, int64_t glim, cudaStream_t stream, Q8Tp wt = Q8Tp{}) {
  if (M <= 0 || K <= 0) return M < 0 || K < 0 ? E_BAD_SHAPE : E_OK;
  const int64_t kpad = round_up(K, 512);
  const int64_t total = M * (kpad / 32);
  const int blocks = (int)((total + 7) / 8 > 148 * 16 ? 148 * 16 : (total + 7) / 8);
  uint8_t* o = static_cast<uint8_t*>(out);
  switch (x_dtype) {
    case DT_F32:
      launch_pdl(quantize_q8_1_kernel<float, MODE>, dim3(blocks), dim3(256), 0, stream, (const float*)x, o, M, K, kpad, sum_mode, ldb, corr_mode, gid, gdiv, glim, wt);
      break;
    case DT_F16:
      launch_pdl(quantize_q8_1_kernel<__half, MODE>, dim3(blocks), dim3(256), 0, stream, (const __half*)x, o, M, K, kpad, sum_mode, ldb, corr_mode, gid, gdiv, glim, wt);
      break;
    case DT_BF16:
      launch_pdl(quantize_q8_1_kernel<__nv_bfloat16, MODE>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)x, o, M, K, kpad, sum_mode, ldb, corr_mode, gid, gdiv, glim, wt);
      break;
    default:
      return E_BAD_DTYPE;
  }
  return cudaGetLastError() == cudaSuccess ? E_OK : E_CUDA;
}

static int launch_f16x8(const void* x, int x_dtype, void* out, int64_t M, int64_t K, int64_t ldb, int corr_mode, int perm,
                        const int32_t* gid, int64_t gdiv, int64_t glim, cudaStream_t stream, int act, int64_t x_ld) {
  if (M <= 0 || K <= 0) return M < 0 || K < 0 ? E_BAD_SHAPE : E_OK;
  const int64_t kpad = round_up(K, 512);
  const int64_t total = M * (kpad / 32);
  const int64_t want = (total + 63) / 64;                 // 64 blocks of 32 per CTA pass
  const int blocks = (int)(want > 148 * 8 ? 148 * 8 : want);
  __half* o = static_cast<__half*>(out);
  switch (x_dtype) {
    case DT_F32:
      launch_pdl(quantize_f16x8_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)x, o, M, K, kpad, ldb, corr_mode, perm, gid, gdiv, glim, act, x_ld);
      break;
    case DT_F16:
      launch_pdl(quantize_f16x8_kernel<__half>, dim3(blocks), dim3(256), 0, stream, (const __half*)x, o, M, K, kpad, ldb, corr_mode, perm, gid, gdiv, glim, act, x_ld);
      break;
    case DT_BF16:
      launch_pdl(quantize_f16x8_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)x, o, M, K, kpad, ldb, corr_mode, perm, gid, gdiv, glim, act, x_ld);
      break;
    default:
      return E_BAD_DTYPE;
  }
  return cudaGetLastError() == cudaSuccess ? E_OK : E_CUDA;
}

int launch_quantize_q8_1(const void* x, int x_dtype, void* out, int64_t M, int64_t K, int mode, int sum_mode,
                         int64_t ldb, int corr_mode, const int32_t* gather_ids, int64_t gather_div, int64_t gather_limit,
                         cudaStream_t stream, int perm, const Q8Tp* wait, int act, int64_t x_ld) {
  if (mode == Q8_MODE_F16) {
    // rows of x and of the output start on 16-byte boundaries when K and ldb are multiples of 8
    const bool aligned = K % 8 == 0 && ldb % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
    if (aligned) return launch_f16x8(x, x_dtype, out, M, K, ldb, corr_mode, perm, gather_ids, gather_div, gather_limit, stream, act, x_ld);
    if (perm || act) return E_BAD_POINTER;
  } else if (act) {
    return E_BAD_SHAPE;
  }
  switch (mode) {
    case Q8_MODE_REF: return launch_mode<Q8_MODE_REF>(x, x_dtype, out, M, K, sum_mode, ldb, corr_mode, nullptr, 1, 0, stream);
    case Q8_MODE_SOA: return launch_mode<Q8_MODE_SOA>(x, x_dtype, out, M, K, sum_mode, ldb, corr_mode, nullptr, 1, 0, stream, wait ? *wait : Q8Tp{});
    case Q8_MODE_F16:
      return launch_mode<Q8_MODE_F16>(x, x_dtype, out, M, K, sum_mode, ldb, corr_mode, gather_ids, gather_div, gather_limit, stream);
  }
  return E_BAD_SHAPE;
}

}  // namespace gguf_b200
