// Standalone dequantize: packed GGUF blocks -> dense fp16/bf16/fp32, bit-identical to the
// reference's ggml_dequantize (vllm_gguf_plugin/csrc/gguf/gguf_kernel.cu:87-102 and the
// per-type kernels of dequantize.cuh:3-15, 69-99, 165-196, 232-256, 258-275, 420-435; further
// types: Q4_1 :17-31, Q5_0 :33-50, Q5_1 :52-69, Q2_K :101-120, Q3_K :122-154, Q5_K :198-230,
// IQ4_NL :400-418).
//
// The reference spends one 32/64-thread CTA per super-block with 1-2 byte loads and strided
// 2-byte stores, and zero-fills the output first.  Here the op is treated as what it is -- an
// output-write-bound stream (2-4 bytes written per 0.26-1.06 bytes read): a persistent grid
// (multiple of the SM count), every lane produces eight consecutive outputs and writes them
// with one 16-byte store (two for fp32), so a warp emits 512 contiguous bytes per step.
//
// Arithmetic is kept step-for-step equal to the reference so that every rounding happens in
// the same place: Q4_0/Q8_0/Q4_K/Q6_K decode in IEEE half (one rounding per multiply or
// subtract; bf16/fp32 outputs are the *half* result converted afterwards), IQ2_XXS/IQ4_XS
// decode in fp32 and round once on the store.
#include "common.cuh"
#include "kernels.h"
#include "tables.cuh"

namespace gguf_b200 {

template <typename out_t> struct Store8;
template <> struct Store8<__half> {
  static __device__ __forceinline__ void st(__half* p, const __half (&h)[8], const float (&)[8], bool from_half) {
    (void)from_half;
    uint4 v;
    v.x = (uint32_t)__half_as_ushort(h[0]) | ((uint32_t)__half_as_ushort(h[1]) << 16);
    v.y = (uint32_t)__half_as_ushort(h[2]) | ((uint32_t)__half_as_ushort(h[3]) << 16);
    v.z = (uint32_t)__half_as_ushort(h[4]) | ((uint32_t)__half_as_ushort(h[5]) << 16);
    v.w = (uint32_t)__half_as_ushort(h[6]) | ((uint32_t)__half_as_ushort(h[7]) << 16);
    *reinterpret_cast<uint4*>(p) = v;
  }
};
template <> struct Store8<__nv_bfloat16> {
  static __device__ __forceinline__ void st(__nv_bfloat16* p, const __half (&)[8], const float (&f)[8], bool) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
      w[i] = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(f[2 * i])) |
             ((uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(f[2 * i + 1])) << 16);
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  }
};
template <> struct Store8<float> {
  static __device__ __forceinline__ void st(float* p, const __half (&)[8], const float (&f)[8], bool) {
    reinterpret_cast<float4*>(p)[0] = make_float4(f[0], f[1], f[2], f[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(f[4], f[5], f[6], f[7]);
  }
};

// Eight outputs produced in half arithmetic: 16-bit-float destinations other than half and
// fp32 destinations receive the half value converted (convert_from_half, ggml-common.h:1079-1096).
template <typename out_t>
__device__ __forceinline__ void store_from_half(out_t* p, const __half (&h)[8]) {
  float f[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) f[i] = __half2float(h[i]);
  Store8<out_t>::st(p, h, f, true);
}
// Eight outputs produced in fp32: rounded once by the store.
template <typename out_t>
__device__ __forceinline__ void store_from_float(out_t* p, const float (&f)[8]) {
  __half h[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) h[i] = __float2half_rn(f[i]);
  Store8<out_t>::st(p, h, f, false);
}

__device__ __forceinline__ uint32_t ldg_u16(const uint8_t* p) { return __ldg(reinterpret_cast<const uint16_t*>(p)); }
// eight bytes from a 2-byte-aligned global address
__device__ __forceinline__ uint2 ldg_8_a2(const uint8_t* p) {
  uint2 r;
  r.x = ldg_u16(p) | (ldg_u16(p + 2) << 16);
  r.y = ldg_u16(p + 4) | (ldg_u16(p + 6) << 16);
  return r;
}
__device__ __forceinline__ uint32_t byte_of(uint2 v, int j) { return ((j < 4 ? v.x : v.y) >> (8 * (j & 3))) & 0xffu; }

__device__ __forceinline__ __half hmul_rn(__half a, __half b) { return __hmul_rn(a, b); }

// Small integers as exact half pairs without an int->half conversion: 0x6400 | n is the half
// 1024 + n (n < 1024), so (w & 0x000F000F) | 0x64006400 holds 1024 + (bits 0-3) and 1024 + (bits 16-19)
// and one exact subtraction leaves the integers.  Two values per instruction instead of one I2F each:
// the kernel was bound by instruction issue (70 % of the issue slots at 0.62 of the memory rate).
// A word of four codes b0..b3 gives the pairs (b0, b2) and (b1, b3); put4 restores the order.
__device__ __forceinline__ __half2 u32_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }
__device__ __forceinline__ __half2 ints_h2(uint32_t two_codes_16_apart, float bias) {   // codes - (bias - 1024), exactly
  return __hsub2_rn(u32_h2(two_codes_16_apart | 0x64006400u), __floats2half2_rn(bias, bias));
}
__device__ __forceinline__ void put4(__half (&h)[8], int base, __half2 a, __half2 b) {
  h[base] = __low2half(a); h[base + 1] = __low2half(b); h[base + 2] = __high2half(a); h[base + 3] = __high2half(b);
}

// d1*q - m1 in half.  The reference writes __hsub(__hmul(d1,q), m1) (dequantize.cuh:193-194)
// with intrinsics that carry no rounding qualifier, which lets the assembler contract the
// pair into one fused multiply-subtract.  CONTRACT selects the fused form explicitly; the
// other form pins two roundings.  The GPU parity test against the reference binary shows it
// uses the fused form on sm_100a; that is the default (gguf_b200_set_q4k_contract).
template <bool CONTRACT> __device__ __forceinline__ __half q4k_value(__half d1, __half q, __half m1) {
  if (CONTRACT) return __hfma(d1, q, __hneg(m1));
  return __hsub_rn(__hmul_rn(d1, q), m1);
}
template <bool CONTRACT> __device__ __forceinline__ __half2 q4k_value2(__half2 d1, __half2 q, __half2 m1) {
  if (CONTRACT) return __hfma2(d1, q, __hneg2(m1));
  return __hsub2_rn(__hmul2_rn(d1, q), m1);
}
// q*d + m of Q4_1 / Q5_1 (__hadd2(__hmul2(v, d), m), dequantize.cuh:28-29, 66-67): the same question
template <bool CONTRACT> __device__ __forceinline__ __half mul_add_value(__half q, __half d, __half m) {
  if (CONTRACT) return __hfma(q, d, m);
  return __hadd_rn(__hmul_rn(q, d), m);
}
__device__ __forceinline__ uint32_t ldg_u32_a2(const uint8_t* p) { return ldg_u16(p) | (ldg_u16(p + 2) << 16); }

// Row gather (embedding look-up: the reference selects the rows with index_select and then
// dequantizes the copy, quantization/vocal_embeds.py:88-96): output row r = weight row ids[r].
struct RowGather {
  const int64_t* ids = nullptr;   // null: plain dequantize of consecutive blocks
  int64_t row_bytes = 0, weight_rows = 0;
  int chunks_per_row = 0;         // K / 256
};

template <int TYPE, typename out_t, bool Q4K_CONTRACT>
__global__ void __launch_bounds__(256) dequantize_kernel(const uint8_t* __restrict__ w_all, out_t* __restrict__ y,
                                                         int64_t n_elems, RowGather rg) {
  __shared__ uint64_t s_grid[TYPE == T_IQ2_XXS ? 256 : 1];
  __shared__ uint8_t s_signs[TYPE == T_IQ2_XXS ? 128 : 1];
  __shared__ int8_t s_kv[16];
  if (TYPE == T_IQ4_XS || TYPE == T_IQ4_NL) {
    if (threadIdx.x < 16) s_kv[threadIdx.x] = d_kvalues_iq4nl[threadIdx.x];
    __syncthreads();
  }
  if (TYPE == T_IQ2_XXS) {
    for (int i = threadIdx.x; i < 256; i += blockDim.x) s_grid[i] = d_iq2xxs_grid[i];
    for (int i = threadIdx.x; i < 128; i += blockDim.x) s_signs[i] = d_ksigns_iq2xs[i];
    __syncthreads();
  }
  constexpr int TS = BlockTraits<TYPE>::TS;
  const int lane = threadIdx.x & 31;
  const int64_t chunks = (n_elems + 255) / 256;  // 256 outputs per warp step
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  // (Two chunks per pass, to have two load chains in flight per warp, measured slower on every type:
  //  Q4_K 14336x4096 32.9 -> 37.4 us.)
  for (int64_t cg = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); cg < chunks; cg += warps) {
    const int64_t o = cg * 256 + lane * 8;
    if (o >= n_elems) continue;
    __half h[8];
    float f[8];
    // chunk c of the block stream that starts at w (gather: the chunk's own weight row)
    const uint8_t* w = w_all;
    int64_t c = cg;
    if (rg.ids) {
      const int64_t r = cg / rg.chunks_per_row, id = rg.ids[r];
      c = cg - r * rg.chunks_per_row;
      if (id < 0 || id >= rg.weight_rows) {   // no such row: zeros (index_select would have refused)
#pragma unroll
        for (int j = 0; j < 8; ++j) { h[j] = __float2half_rn(0.f); f[j] = 0.f; }
        Store8<out_t>::st(y + o, h, f, false);
        continue;
      }
      w = w_all + id * rg.row_bytes;
    }
    if (TYPE == T_Q4_0) {  // dequantize_q4_0: (q - 8) exactly, then one half multiply by d
      const uint8_t* blk = w + (c * 8 + (lane >> 2)) * TS;
      const __half d = __ushort_as_half((unsigned short)ldg_u16(blk));
      const uint2 q = ldg_8_a2(blk + 2 + 8 * (lane & 1));
      const int sh = (lane & 2) ? 4 : 0;
      const __half2 d2 = __half2half2(d);
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const uint32_t ws = (i ? q.y : q.x) >> sh;
        put4(h, 4 * i, __hmul2_rn(ints_h2(ws & 0x000F000Fu, 1032.f), d2), __hmul2_rn(ints_h2((ws >> 8) & 0x000F000Fu, 1032.f), d2));
      }
      store_from_half(y + o, h);
    } else if (TYPE == T_Q8_0) {  // dequantize_q8_0
      const uint8_t* blk = w + (c * 8 + (lane >> 2)) * TS;
      const __half d = __ushort_as_half((unsigned short)ldg_u16(blk));
      const uint2 q = ldg_8_a2(blk + 2 + 8 * (lane & 3));
      const __half2 d2 = __half2half2(d);
#pragma unroll
      for (int i = 0; i < 2; ++i) {   // int8 b -> b + 128 (flip the sign bit) -> 1024 + 128 + b -> b
        const uint32_t ws = (i ? q.y : q.x) ^ 0x80808080u;
        put4(h, 4 * i, __hmul2_rn(ints_h2(ws & 0x00FF00FFu, 1152.f), d2), __hmul2_rn(ints_h2((ws >> 8) & 0x00FF00FFu, 1152.f), d2));
      }
      store_from_half(y + o, h);
    } else if (TYPE == T_Q4_K) {  // dequantize_block_q4_K
      const uint8_t* blk = w + c * TS;
      const uint32_t dm = __ldg(reinterpret_cast<const uint32_t*>(blk));
      const __half dall = __ushort_as_half((unsigned short)(dm & 0xffff)), dmin = __ushort_as_half((unsigned short)(dm >> 16));
      const int il = lane >> 3, off = (lane & 7) * 8;       // 64-value group, offset inside it
      const int hi = off >= 32;                               // upper nibbles belong to sub-block 2*il+1
      const int is = 2 * il + hi;
      const uint8_t* sc8 = blk + 4;
      int sc, m;
      if (is < 4) {
        sc = __ldg(sc8 + is) & 63;
        m = __ldg(sc8 + is + 4) & 63;
      } else {
        sc = (__ldg(sc8 + is + 4) & 0xF) | ((__ldg(sc8 + is - 4) >> 6) << 4);
        m = (__ldg(sc8 + is + 4) >> 4) | ((__ldg(sc8 + is) >> 6) << 4);
      }
      const __half d1 = hmul_rn(dall, __int2half_rn(sc)), m1 = hmul_rn(dmin, __int2half_rn(m));
      const uint2 q = __ldg(reinterpret_cast<const uint2*>(blk + 16 + 32 * il + (off & 31)));
      const __half2 d12 = __half2half2(d1), m12 = __half2half2(m1);
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const uint32_t ws = (i ? q.y : q.x) >> (4 * hi);
        put4(h, 4 * i, q4k_value2<Q4K_CONTRACT>(d12, ints_h2(ws & 0x000F000Fu, 1024.f), m12),
             q4k_value2<Q4K_CONTRACT>(d12, ints_h2((ws >> 8) & 0x000F000Fu, 1024.f), m12));
      }
      store_from_half(y + o, h);
    } else if (TYPE == T_Q6_K) {  // dequantize_block_q6_K
      const uint8_t* blk = w + c * TS;
      const int ip = lane >> 4, off = (lane & 15) * 8, qd = off >> 5, l0 = off & 31;
      const uint2 ql = ldg_8_a2(blk + 64 * ip + 32 * (qd & 1) + l0);
      const uint2 qh = ldg_8_a2(blk + 128 + 32 * ip + l0);
      const int sc = (int)(int8_t)__ldg(blk + 192 + 8 * ip + 2 * qd + (l0 >> 4));
      const __half d = __ushort_as_half((unsigned short)ldg_u16(blk + 208));
      // (The pair form used for the 4- and 8-bit types above gained nothing here -- 99.4 vs 98.1 us on
      //  37888x3584 -- and a product of a negative scale with a zero code comes out as -0 where the
      //  reference's integer product gives +0, so the integer form stays.)
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int lo = (byte_of(ql, j) >> (4 * (qd >> 1))) & 0xF;
        const int hb = (byte_of(qh, j) >> (2 * qd)) & 3;
        h[j] = hmul_rn(d, __int2half_rn(sc * ((lo | (hb << 4)) - 32)));
      }
      store_from_half(y + o, h);
    } else if (TYPE == T_IQ2_XXS) {  // dequantize_block_iq2_xxs (fp32)
      const uint8_t* blk = w + c * TS;
      const int ib = lane >> 2, il = lane & 3;
      const uint8_t* q2 = blk + 2 + 8 * ib;
      const uint32_t aux32 = ldg_u16(q2 + 4) | (ldg_u16(q2 + 6) << 16);
      const float d = __half2float(__ushort_as_half((unsigned short)ldg_u16(blk))) * (0.5f + (float)(aux32 >> 28)) * 0.25f;
      const uint64_t grid = s_grid[__ldg(q2 + il)];
      const uint32_t signs = s_signs[(aux32 >> (7 * il)) & 127];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        f[j] = d * (float)((uint32_t)(grid >> (8 * j)) & 0xffu) * ((signs >> j) & 1 ? -1.f : 1.f);
      store_from_float(y + o, f);
    } else if (TYPE == T_IQ2_XS || TYPE == T_IQ2_S || TYPE == T_IQ3_XXS || TYPE == T_IQ3_S) {
      // dequantize_block_iq2_xs / iq2_s / iq3_xxs / iq3_s (dequantize.cuh:277-353): eight values =
      // sub-block scale * code-book magnitudes * signs, all in fp32, one rounding at the store.
      // The code books are read from global memory (this kernel is bound by its stores).
      const uint8_t* blk = w + c * TS;
      const int ib = lane >> 2, il = lane & 3;
      const float dh = __half2float(__ushort_as_half((unsigned short)ldg_u16(blk)));
      uint64_t grid;      // eight magnitudes, byte j = value j
      uint32_t signs;     // bit j set = value j negative
      float d;
      if (TYPE == T_IQ2_XS) {
        const uint32_t q = ldg_u16(blk + 2 + 2 * (4 * ib + il));
        grid = __ldg(&d_iq2xs_grid[q & 511]);
        signs = __ldg(&d_ksigns_iq2xs[q >> 9]);
        d = dh * (0.5f + (float)((__ldg(blk + 66 + ib) >> (4 * (il / 2))) & 0xf)) * 0.25f;
      } else if (TYPE == T_IQ2_S) {
        const uint32_t qh = __ldg(blk + 66 + ib);
        grid = __ldg(&d_iq2s_grid[__ldg(blk + 2 + 4 * ib + il) | ((qh << (8 - 2 * il)) & 0x300)]);
        signs = __ldg(blk + 2 + 32 + 4 * ib + il);
        d = dh * (0.5f + (float)((__ldg(blk + 74 + ib) >> (4 * (il / 2))) & 0xf)) * 0.25f;
      } else if (TYPE == T_IQ3_XXS) {
        const uint8_t* q3 = blk + 2 + 8 * ib;
        const uint32_t aux32 = ldg_u16(blk + 2 + 64 + 4 * ib) | (ldg_u16(blk + 2 + 64 + 4 * ib + 2) << 16);
        grid = (uint64_t)__ldg(&d_iq3xxs_grid[__ldg(q3 + 2 * il)]) | ((uint64_t)__ldg(&d_iq3xxs_grid[__ldg(q3 + 2 * il + 1)]) << 32);
        signs = __ldg(&d_ksigns_iq2xs[(aux32 >> (7 * il)) & 127]);
        d = dh * (0.5f + (float)(aux32 >> 28)) * 0.5f;
      } else {
        const uint8_t* qs = blk + 2 + 8 * ib;
        const uint32_t qh = __ldg(blk + 66 + ib);
        grid = (uint64_t)__ldg(&d_iq3s_grid[__ldg(qs + 2 * il) | ((qh << (8 - 2 * il)) & 256)]) |
               ((uint64_t)__ldg(&d_iq3s_grid[__ldg(qs + 2 * il + 1) | ((qh << (7 - 2 * il)) & 256)]) << 32);
        signs = __ldg(blk + 74 + 4 * ib + il);
        d = dh * (0.5f + (float)((__ldg(blk + 106 + ib / 2) >> (4 * (ib % 2))) & 0xf)) * 0.5f;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j)
        f[j] = d * (float)((uint32_t)(grid >> (8 * j)) & 0xffu) * ((signs >> j) & 1 ? -1.f : 1.f);
      store_from_float(y + o, f);
    } else if (TYPE == T_IQ1_S || TYPE == T_IQ1_M) {
      // dequantize_block_iq1_s / iq1_m (dequantize.cuh:355-399): value = d * (q + delta), q in {0,1,2}
      // from the code book (nibble-packed), delta = -1 -+ 1/8 chosen per group by a bit of qh.
      const uint8_t* blk = w + c * TS;
      const int ib = lane >> 2, il = lane & 3;
      float d, delta;
      uint32_t g;
      if (TYPE == T_IQ1_S) {
        const uint32_t qh = ldg_u16(blk + 34 + 2 * ib);
        delta = (qh & 0x8000) ? -1.f - 0.125f : -1.f + 0.125f;
        d = __half2float(__ushort_as_half((unsigned short)ldg_u16(blk))) * (float)(2 * ((qh >> 12) & 7) + 1);
        g = __ldg(&d_iq1s_grid[__ldg(blk + 2 + 4 * ib + il) | (((qh >> (3 * il)) & 7) << 8)]);
      } else {
        const uint32_t sc0 = ldg_u16(blk + 48), sc1 = ldg_u16(blk + 50), sc2 = ldg_u16(blk + 52), sc3 = ldg_u16(blk + 54);
        const uint32_t s16 = (sc0 >> 12) | ((sc1 >> 8) & 0x00f0) | ((sc2 >> 4) & 0x0f00) | (sc3 & 0xf000);
        const int ib16 = 2 * ib + il / 2;
        const uint32_t scw = ldg_u16(blk + 48 + 2 * (ib16 / 4));
        d = __half2float(__ushort_as_half((unsigned short)s16)) * (float)(2 * ((scw >> (3 * (ib16 % 4))) & 7) + 1);
        const uint32_t qh = __ldg(blk + 32 + 2 * ib + il / 2);
        delta = (qh & (0x08u << (4 * (il % 2)))) ? -1.f - 0.125f : -1.f + 0.125f;
        g = __ldg(&d_iq1s_grid[__ldg(blk + 4 * ib + il) | (((qh >> (4 * (il % 2))) & 7) << 8)]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = d * ((float)((g >> (8 * (j & 3) + 4 * (j >> 2))) & 0xfu) + delta);
      store_from_float(y + o, f);
    } else if (TYPE == T_Q4_1) {  // dequantize_q4_1: q*d + m
      const uint8_t* blk = w + (c * 8 + (lane >> 2)) * TS;
      const uint32_t dm = __ldg(reinterpret_cast<const uint32_t*>(blk));
      const __half d = __ushort_as_half((unsigned short)(dm & 0xffff)), m = __ushort_as_half((unsigned short)(dm >> 16));
      const int sh = (lane & 2) ? 4 : 0;   // (20-byte blocks: 4-byte aligned)
      const uint32_t qa = __ldg(reinterpret_cast<const uint32_t*>(blk + 4 + 8 * (lane & 1))), qb = __ldg(reinterpret_cast<const uint32_t*>(blk + 8 + 8 * (lane & 1)));
#pragma unroll
      for (int j = 0; j < 8; ++j)
        h[j] = mul_add_value<Q4K_CONTRACT>(__int2half_rn((int)((((j < 4 ? qa : qb) >> (8 * (j & 3))) >> sh) & 0xF)), d, m);
      store_from_half(y + o, h);
    } else if (TYPE == T_Q5_0 || TYPE == T_Q5_1) {  // dequantize_q5_0: (q - 16)*d ; dequantize_q5_1: q*d + m
      constexpr int HDR = TYPE == T_Q5_1 ? 4 : 2;
      const uint8_t* blk = w + (c * 8 + (lane >> 2)) * TS;
      const __half d = __ushort_as_half((unsigned short)ldg_u16(blk));
      const __half m = TYPE == T_Q5_1 ? __ushort_as_half((unsigned short)ldg_u16(blk + 2)) : __half();
      const uint32_t qh = ldg_u32_a2(blk + HDR);
      const int t = lane & 3, j0 = 8 * (t & 1);               // values 8t..8t+7: bytes qs[j0..j0+7], low (t < 2) or high nibbles
      const uint2 q = ldg_8_a2(blk + HDR + 4 + j0);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int b = byte_of(q, j), jj = j0 + j;
        const int x = t < 2 ? ((b & 0xF) | (int)(((qh >> jj) << 4) & 0x10)) : ((b >> 4) | (int)((qh >> (jj + 12)) & 0x10));
        if (TYPE == T_Q5_1) h[j] = mul_add_value<Q4K_CONTRACT>(__int2half_rn(x), d, m);
        else h[j] = hmul_rn(__hsub_rn(__int2half_rn(x), __int2half_rn(16)), d);
      }
      store_from_half(y + o, h);
    } else if (TYPE == T_IQ4_NL) {  // dequantize_block_iq4_nl (fp32)
      const uint8_t* blk = w + (c * 8 + (lane >> 2)) * TS;
      const float d = __half2float(__ushort_as_half((unsigned short)ldg_u16(blk)));
      const uint2 q = ldg_8_a2(blk + 2 + 8 * (lane & 1));
      const int sh = (lane & 2) ? 4 : 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = d * (float)s_kv[(byte_of(q, j) >> sh) & 0xF];
      store_from_float(y + o, f);
    } else if (TYPE == T_Q2_K) {  // dequantize_block_q2_K
      const uint8_t* blk = w + c * TS;                         // 84-byte blocks: 4-byte aligned
      const int v = 8 * lane, n = v >> 7, k = (v & 127) >> 5, l0 = v & 31;
      const int sc = __ldg(blk + 8 * n + (l0 >> 4) + 2 * k);
      const uint32_t dm = __ldg(reinterpret_cast<const uint32_t*>(blk + 80));
      const __half dall = __ushort_as_half((unsigned short)(dm & 0xffff)), dmin = __ushort_as_half((unsigned short)(dm >> 16));
      const __half mm = hmul_rn(dmin, __int2half_rn(sc >> 4));
      const uint32_t qa = __ldg(reinterpret_cast<const uint32_t*>(blk + 16 + 32 * n + l0)), qb = __ldg(reinterpret_cast<const uint32_t*>(blk + 20 + 32 * n + l0));
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int q2 = (((j < 4 ? qa : qb) >> (8 * (j & 3))) >> (2 * k)) & 3;
        h[j] = q4k_value<Q4K_CONTRACT>(dall, __int2half_rn((sc & 0xF) * q2), mm);
      }
      store_from_half(y + o, h);
    } else if (TYPE == T_Q3_K) {  // dequantize_block_q3_K
      const uint8_t* blk = w + c * TS;                         // 110-byte blocks: 2-byte aligned
      const int v = 8 * lane, n = v >> 7, jq = (v & 127) >> 5, l0 = v & 31, is = 8 * n + 2 * jq + (l0 >> 4);
      const uint8_t* scp = blk + 96;
      int us;
      if (is < 4) us = (__ldg(scp + is) & 0xF) | (((__ldg(scp + is + 8) >> 0) & 3) << 4);
      else if (is < 8) us = (__ldg(scp + is) & 0xF) | (((__ldg(scp + is + 4) >> 2) & 3) << 4);
      else if (is < 12) us = (__ldg(scp + is - 8) >> 4) | (((__ldg(scp + is) >> 4) & 3) << 4);
      else us = (__ldg(scp + is - 8) >> 4) | (((__ldg(scp + is - 4) >> 6) & 3) << 4);
      const __half dl = hmul_rn(__ushort_as_half((unsigned short)ldg_u16(blk + 108)), __int2half_rn((int)(int8_t)us - 32));
      const uint2 q = ldg_8_a2(blk + 32 + 32 * n + l0), hm = ldg_8_a2(blk + l0);
      const int mbit = 1 << (4 * n + jq);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int x = (int)((byte_of(q, j) >> (2 * jq)) & 3) - ((byte_of(hm, j) & mbit) ? 0 : 4);
        h[j] = hmul_rn(dl, __int2half_rn(x));
      }
      store_from_half(y + o, h);
    } else if (TYPE == T_Q5_K) {  // dequantize_block_q5_K
      const uint8_t* blk = w + c * TS;                         // 176-byte blocks: 16-byte aligned
      const uint32_t dm = __ldg(reinterpret_cast<const uint32_t*>(blk));
      const __half dall = __ushort_as_half((unsigned short)(dm & 0xffff)), dmin = __ushort_as_half((unsigned short)(dm >> 16));
      const int il = lane >> 3, off = (lane & 7) * 8, hi = off >= 32, l0 = off & 31, is = 2 * il + hi;
      const uint8_t* sc8 = blk + 4;
      int sc, m;
      if (is < 4) {
        sc = __ldg(sc8 + is) & 63;
        m = __ldg(sc8 + is + 4) & 63;
      } else {
        sc = (__ldg(sc8 + is + 4) & 0xF) | ((__ldg(sc8 + is - 4) >> 6) << 4);
        m = (__ldg(sc8 + is + 4) >> 4) | ((__ldg(sc8 + is) >> 6) << 4);
      }
      const __half d1 = hmul_rn(dall, __int2half_rn(sc)), m1 = hmul_rn(dmin, __int2half_rn(m));
      const uint2 q = __ldg(reinterpret_cast<const uint2*>(blk + 48 + 32 * il + l0));
      const uint2 qh = __ldg(reinterpret_cast<const uint2*>(blk + 16 + l0));
      const int hbit = 1 << (2 * il + hi);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int x = (int)((byte_of(q, j) >> (4 * hi)) & 0xF) + ((byte_of(qh, j) & hbit) ? 16 : 0);
        h[j] = q4k_value<Q4K_CONTRACT>(d1, __int2half_rn(x), m1);
      }
      store_from_half(y + o, h);
    } else {  // T_IQ4_XS: dequantize_block_iq4_xs (fp32)
      const uint8_t* blk = w + c * TS;
      const int ib = lane >> 2, off = (lane & 3) * 8, hi = off >= 16;
      const uint32_t sh = ldg_u16(blk + 2);
      const int ls = ((__ldg(blk + 4 + ib / 2) >> (4 * (ib & 1))) & 0xf) | (((sh >> (2 * ib)) & 3) << 4);
      const float d = __half2float(__ushort_as_half((unsigned short)ldg_u16(blk))) * (float)(ls - 32);
      const uint2 q = __ldg(reinterpret_cast<const uint2*>(blk + 8 + 16 * ib + (off & 15)));
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = d * (float)s_kv[(byte_of(q, j) >> (4 * hi)) & 0xF];
      store_from_float(y + o, f);
    }
  }
}

template <int TYPE, typename out_t>
static int launch_t(const void* w, void* out, int64_t n, int q4k_contract, cudaStream_t s, const RowGather& rg) {
  const int64_t chunks = (n + 255) / 256;
  int64_t ctas = (chunks + 7) / 8;
  const int64_t cap = 148 * 32;  // four rounds of the 8 resident CTAs per SM measured best (148*8: -5 %, one CTA per 8 chunks: -25 %)
  if (ctas > cap) ctas = cap;
  if (ctas < 1) ctas = 1;
  constexpr bool fusible = TYPE == T_Q4_K || TYPE == T_Q5_K || TYPE == T_Q2_K || TYPE == T_Q4_1 || TYPE == T_Q5_1;
  if (fusible && q4k_contract)
    dequantize_kernel<TYPE, out_t, true><<<(int)ctas, 256, 0, s>>>((const uint8_t*)w, (out_t*)out, n, rg);
  else
    dequantize_kernel<TYPE, out_t, false><<<(int)ctas, 256, 0, s>>>((const uint8_t*)w, (out_t*)out, n, rg);
  return cudaGetLastError() == cudaSuccess ? E_OK : E_CUDA;
}

template <int TYPE>
static int launch_d(const void* w, void* out, int dt, int64_t n, int c, cudaStream_t s, const RowGather& rg) {
  switch (dt) {
    case DT_F32: return launch_t<TYPE, float>(w, out, n, c, s, rg);
    case DT_F16: return launch_t<TYPE, __half>(w, out, n, c, s, rg);
    case DT_BF16: return launch_t<TYPE, __nv_bfloat16>(w, out, n, c, s, rg);
  }
  return E_BAD_DTYPE;
}

int launch_dequantize(const void* w, int type, void* out, int out_dtype, int64_t n_elems, int q4k_contract,
                      cudaStream_t stream, const int64_t* row_ids, int64_t K, int64_t weight_rows) {
  if (n_elems == 0) return E_OK;
  RowGather rg;
  if (row_ids) {
    rg.ids = row_ids;
    rg.row_bytes = K / dequant_block_size(type) * dequant_type_size(type);
    rg.weight_rows = weight_rows;
    rg.chunks_per_row = (int)(K / 256);
  }
  switch (type) {
    case T_Q4_0: return launch_d<T_Q4_0>(w, out, out_dtype, n_elems, q4k_contract, stream, rg);
    case T_Q8_0: return launch_d<T_Q8_0>(w, out, out_dtype, n_elems, q4k_contract, stream, rg);
    case T_Q4_K: return launch_d<T_Q4_K>(w, out, out_dtype, n_elems, q4k_contract, stream, rg);
    case T_Q6_K: return launch_d<T_Q6_K>(w, out, out_dtype, n_elems, q4k_contract, stream, rg);
    case T_IQ2_XXS: return launch_d<T_IQ2_XXS>(w, out, out_dtype, n_elems, q4k_contract, stream, rg);
    case T_IQ4_XS: return launch_d<T_IQ4_XS>(w, out, out_dtype, n_elems, q4k_contract, stream, rg);
    case T_Q4_1: return launch_d<T_Q4_1>(w, out, out_dtype, n_elems, q4k_contract, stream, rg);
    case T_Q5_0: return launch_d<T_Q5_0>(w, out, out_dtype, n_elems, q4k_contract, stream, rg);
    case T_Q5_1: return launch_d<T_Q5_1>(w, out, out_dtype, n_elems, q4k_contract, stream, rg);
    case T_Q2_K: return launch_d<T_Q2_K>(w, out, out_dtype, n_elems, q4k_contract, stream, rg);
    case T_Q3_K: return launch_d<T_Q3_K>(w, out, out_dtype, n_elems, q4k_contract, stream, rg);
    case T_Q5_K: return launch_d<T_Q5_K>(w, out, out_dtype, n_elems, q4k_contract, stream, rg);
    case T_IQ4_NL: return launch_d<T_IQ4_NL>(w, out, out_dtype, n_elems, q4k_contract, stream, rg);
    case T_IQ2_XS: return launch_d<T_IQ2_XS>(w, out, out_dtype, n_elems, q4k_contract, stream, rg);
    case T_IQ2_S: return launch_d<T_IQ2_S>(w, out, out_dtype, n_elems, q4k_contract, stream, rg);
    case T_IQ3_XXS: return launch_d<T_IQ3_XXS>(w, out, out_dtype, n_elems, q4k_contract, stream, rg);
    case T_IQ3_S: return launch_d<T_IQ3_S>(w, out, out_dtype, n_elems, q4k_contract, stream, rg);
    case T_IQ1_S: return launch_d<T_IQ1_S>(w, out, out_dtype, n_elems, q4k_contract, stream, rg);
    case T_IQ1_M: return launch_d<T_IQ1_M>(w, out, out_dtype, n_elems, q4k_contract, stream, rg);
  }
  return E_BAD_TYPE;
}

}  // namespace gguf_b200
