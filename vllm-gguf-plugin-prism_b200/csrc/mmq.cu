// Prefill GEMM on the 5th-generation tensor cores:  D[n, t] = sum_k A[n, k] * B[t, k]
// with A = weight tile decoded on the fly from packed GGUF blocks and B = activations.
// Serves three entry points:
//   * ggml_mul_mat_a8   (reference: gguf_kernel.cu:220-290 + mul_mat_q, mmq.cuh:2-104)
//   * ggml_moe_a8       (reference: gguf_kernel.cu:292-393 + moe_q, moe.cuh:5-129)
//   * dequantize-then-matmul of the IQ types (reference: quantization/linear.py:50-54)
//
// Why fp16 operands and not int8: the contraction carries a different fp scale per 32
// values on BOTH operands (weights: d or d*sc; activations: the q8_1 d).  An int8 MMA would
// have to drain its int32 accumulator and rescale it on the CUDA cores after every K=32 step
// (128 x 256 accumulators per ~130 tensor clocks), which bounds it near 10-25 % of int8 peak.
// Folding the scales into the operands instead -- A = half(scale * code) decoded exactly as
// the reference's own dequantize does, B = half(d8 * q8) from the bit-exact q8_1 quantizer --
// keeps ONE fp32 accumulator in tensor memory over the whole K with no drain, at the price of
// one fp16 rounding per operand (~3e-4 relative L2, far inside the 2e-3 budget).  The q8_1
// "sum" terms the reference's tiled kernels use (Q4_0: -8*d*s8, Q4_K: -dmin*m*s8, with s8 the
// fp16 sum of the *unquantized* activations) ride along as K/32 extra contraction columns.
//
// Tile: 128 weight rows (UMMA M) x TN tokens (UMMA N, 16..256) x 64 values per stage, both
// operands K-major in shared memory with the 128-byte swizzle.  Weight rows sit on the M axis
// so that small token counts (M = 8, MoE blocks) do not waste the 128-row instruction.
// Warp roles:  warps 0-3 decode weights into the A stage (one row per thread) and later run
// the epilogue (tcgen05.ld, one TMEM lane = one weight row per thread); warp 4 issues the TMA
// loads of the B tile (tiled 2-D tensor map, no multicast) and owns the TMEM allocation;
// warp 5 lane 0 issues tcgen05.mma and commits stage releases.  A 4-deep mbarrier ring
// decouples them.  Every wait is bounded and reports through the status word.
#include <cuda.h>

#include <type_traits>

#include "common.cuh"
#include "kernels.h"
#include "tables.cuh"

namespace gguf_b200 {

constexpr int MMQ_ROWS = 128;
constexpr int MMQ_BK = 64;
constexpr int MMQ_STAGES = 4;
constexpr int MMQ_THREADS = 192;
constexpr int MMQ_A_STAGE = MMQ_ROWS * MMQ_BK * 2;  // 16 KB

// ---- tcgen05 wrappers -------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* slot_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot_smem)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

// K-major, 128-byte swizzle: rows of 128 B, 8-row groups 1024 B apart (stride byte offset),
// leading byte offset unused by swizzled K-major layouts (1), descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// kind::f16 instruction descriptor: fp32 accumulator, A/B format (0 = f16, 1 = bf16), both K-major
__host__ __device__ inline uint32_t umma_idesc(int m, int n, int fmt) {
  return (1u << 4) | ((uint32_t)fmt << 7) | ((uint32_t)fmt << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// ---- weight decoders: 64 consecutive values of one row -> 32 packed 16-bit pairs --------

template <typename ab_t> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  return (uint32_t)__half_as_ushort(__float2half_rn(a)) | ((uint32_t)__half_as_ushort(__float2half_rn(b)) << 16);
}
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(a)) | ((uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(b)) << 16);
}
__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }
// (1024 + a, 1024 + b) as half2 for small unsigned a, b: exact integers, so subtracting
// 1024 + bias afterwards yields (a - bias, b - bias) without any rounding.
__device__ __forceinline__ __half2 ints_plus_1024(uint32_t a, uint32_t b) { return u32_as_h2(0x64006400u | a | (b << 16)); }
__device__ __forceinline__ __half2 hmul2_rn(__half2 a, __half2 b) { return __hmul2_rn(a, b); }

__device__ __forceinline__ uint32_t ldg16(const uint8_t* p) { return __ldg(reinterpret_cast<const uint16_t*>(p)); }

struct DecodeCtx {
  const uint64_t* grid;   // IQ2_XXS tables in shared memory
  const uint8_t* signs;
  const int8_t* kv;       // IQ4_XS levels in shared memory
};

template <int TYPE, typename ab_t> struct Decoder;

// Q4_0: value = half((q - 8) * d), dequantize_q4_0 (dequantize.cuh:3-15)
template <typename ab_t> struct Decoder<T_Q4_0, ab_t> {
  static __device__ __forceinline__ void slab(const uint8_t* row, int s, int64_t K, const DecodeCtx&, uint32_t (&out)[32]) {
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      const int64_t blk_i = 2 * (int64_t)s + b;
      if (blk_i * 32 >= K) {
#pragma unroll
        for (int i = 0; i < 16; ++i) out[16 * b + i] = 0;
        continue;
      }
      const uint8_t* blk = row + blk_i * 18;
      const uint32_t du = ldg16(blk);
      const __half2 d2 = u32_as_h2(du | (du << 16));
      const __half2 off = __floats2half2_rn(1032.f, 1032.f);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint32_t t = ldg16(blk + 2 + 2 * i);  // qs[2i], qs[2i+1]
        out[16 * b + i] = h2_as_u32(hmul2_rn(__hsub2(ints_plus_1024(t & 0xF, (t >> 8) & 0xF), off), d2));
        out[16 * b + 8 + i] = h2_as_u32(hmul2_rn(__hsub2(ints_plus_1024((t >> 4) & 0xF, (t >> 12) & 0xF), off), d2));
      }
    }
  }
  // correction columns: A'[n, g] = d of block g (pairs with 8*(d8*sum(q8) - s8) on the B side)
  static __device__ __forceinline__ void corr(const uint8_t* row, int c, int64_t K, uint32_t (&out)[32]) {
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const int64_t g = 64 * (int64_t)c + 2 * i;
      const uint32_t a = g * 32 < K ? ldg16(row + g * 18) : 0u;
      const uint32_t b = (g + 1) * 32 < K ? ldg16(row + (g + 1) * 18) : 0u;
      out[i] = a | (b << 16);
    }
  }
};

// Q8_0: value = half(q * d), dequantize_q8_0 (dequantize.cuh:69-78)
template <typename ab_t> struct Decoder<T_Q8_0, ab_t> {
  static __device__ __forceinline__ void slab(const uint8_t* row, int s, int64_t K, const DecodeCtx&, uint32_t (&out)[32]) {
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      const int64_t blk_i = 2 * (int64_t)s + b;
      if (blk_i * 32 >= K) {
#pragma unroll
        for (int i = 0; i < 16; ++i) out[16 * b + i] = 0;
        continue;
      }
      const uint8_t* blk = row + blk_i * 34;
      const uint32_t du = ldg16(blk);
      const __half2 d2 = u32_as_h2(du | (du << 16));
      const __half2 off = __floats2half2_rn(1152.f, 1152.f);  // 1024 + 128
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const uint32_t t = ldg16(blk + 2 + 2 * i) ^ 0x8080u;  // int8 -> biased unsigned
        out[16 * b + i] = h2_as_u32(hmul2_rn(__hsub2(ints_plus_1024(t & 0xFF, t >> 8), off), d2));
      }
    }
  }
  static __device__ __forceinline__ void corr(const uint8_t*, int, int64_t, uint32_t (&)[32]) {}
};

// 6-bit (scale, min) pair j of a Q4_K super-block from its 12 packed bytes held in three
// registers (bytes 0-3, 4-7, 8-11); same packing as get_scale_min_k4, dequantize.cuh:156-163.
__device__ __forceinline__ void q4k_scale_min(uint32_t w0, uint32_t w1, uint32_t w2, int j, int& sc, int& m) {
  if (j < 4) {
    sc = (w0 >> (8 * j)) & 63;
    m = (w1 >> (8 * j)) & 63;
  } else {
    const int sh = 8 * (j - 4);
    const uint32_t b = (w2 >> sh) & 0xFF;
    sc = (b & 0xF) | ((((w0 >> sh) & 0xFF) >> 6) << 4);
    m = (b >> 4) | ((((w1 >> sh) & 0xFF) >> 6) << 4);
  }
}

// Q4_K: A = half(d1 * q) with d1 = half(d * sc); the -dmin*m part is a correction column
template <typename ab_t> struct Decoder<T_Q4_K, ab_t> {
  static __device__ __forceinline__ void slab(const uint8_t* row, int s, int64_t, const DecodeCtx&, uint32_t (&out)[32]) {
    const uint8_t* blk = row + (int64_t)(s >> 2) * 144;
    const int p = s & 3;
    const uint4 hdr = __ldg(reinterpret_cast<const uint4*>(blk));
    const __half dall = __ushort_as_half((unsigned short)(hdr.x & 0xffff));
    int sc0, sc1, m0, m1;
    q4k_scale_min(hdr.y, hdr.z, hdr.w, 2 * p, sc0, m0);
    q4k_scale_min(hdr.y, hdr.z, hdr.w, 2 * p + 1, sc1, m1);
    (void)m0;
    (void)m1;
    const __half d1 = __hmul_rn(dall, __int2half_rn(sc0)), d2 = __hmul_rn(dall, __int2half_rn(sc1));
    const __half2 d1v = __half2half2(d1), d2v = __half2half2(d2);
    const __half2 off = __floats2half2_rn(1024.f, 1024.f);
    const uint4* qp = reinterpret_cast<const uint4*>(blk + 16 + 32 * p);
    const uint4 qa = __ldg(qp), qb = __ldg(qp + 1);
    const uint32_t q[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {  // word i: bytes 4i..4i+3 -> values 4i.. (low nibbles) and 32+4i.. (high)
      const uint32_t w = q[i];
      out[2 * i] = h2_as_u32(hmul2_rn(__hsub2(ints_plus_1024(w & 0xF, (w >> 8) & 0xF), off), d1v));
      out[2 * i + 1] = h2_as_u32(hmul2_rn(__hsub2(ints_plus_1024((w >> 16) & 0xF, (w >> 24) & 0xF), off), d1v));
      out[16 + 2 * i] = h2_as_u32(hmul2_rn(__hsub2(ints_plus_1024((w >> 4) & 0xF, (w >> 12) & 0xF), off), d2v));
      out[16 + 2 * i + 1] = h2_as_u32(hmul2_rn(__hsub2(ints_plus_1024((w >> 20) & 0xF, (w >> 28) & 0xF), off), d2v));
    }
  }
  // correction columns: A'[n, g] = half(dmin * m_g)  (pairs with -s8 on the B side)
  static __device__ __forceinline__ void corr(const uint8_t* row, int c, int64_t K, uint32_t (&out)[32]) {
#pragma unroll
    for (int sb = 0; sb < 8; ++sb) {
      const int64_t sbi = 8 * (int64_t)c + sb;  // super-block index: 8 groups each
      if (sbi * 256 >= K) {
#pragma unroll
        for (int i = 0; i < 4; ++i) out[4 * sb + i] = 0;
        continue;
      }
      const uint8_t* blk = row + sbi * 144;
      const uint4 hdr = __ldg(reinterpret_cast<const uint4*>(blk));
      const __half dmin = __ushort_as_half((unsigned short)(hdr.x >> 16));
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        int sc, ma, mb;
        q4k_scale_min(hdr.y, hdr.z, hdr.w, 2 * i, sc, ma);
        q4k_scale_min(hdr.y, hdr.z, hdr.w, 2 * i + 1, sc, mb);
        out[4 * sb + i] = (uint32_t)__half_as_ushort(__hmul_rn(dmin, __int2half_rn(ma))) |
                          ((uint32_t)__half_as_ushort(__hmul_rn(dmin, __int2half_rn(mb))) << 16);
      }
    }
  }
};

// Q6_K: value = half(d * half(sc * (code - 32))), dequantize_block_q6_K (dequantize.cuh:232-256)
template <typename ab_t> struct Decoder<T_Q6_K, ab_t> {
  static __device__ __forceinline__ void slab(const uint8_t* row, int s, int64_t, const DecodeCtx&, uint32_t (&out)[32]) {
    const uint8_t* blk = row + (int64_t)(s >> 2) * 210;
    const int ip = (s >> 1) & 1, odd = s & 1;
    const uint32_t du = ldg16(blk + 208);
    const __half2 d2 = u32_as_h2(du | (du << 16));
    const __half2 off = __floats2half2_rn(1056.f, 1056.f);  // 1024 + 32
    const uint8_t* ql = blk + 64 * ip;
    const uint8_t* qh = blk + 128 + 32 * ip;
    const int8_t* sc = reinterpret_cast<const int8_t*>(blk + 192 + 8 * ip + 4 * odd);
#pragma unroll
    for (int i = 0; i < 32; ++i) {  // pair i: values 2i, 2i+1 of the slab
      const int j = 2 * i;          // ql byte index 64ip + j; qh byte 32ip + j%32, shift 2q, q = 2*odd + j/32
      const uint32_t l = ldg16(ql + j) >> (4 * odd);
      const uint32_t h = ldg16(qh + (j & 31)) >> (2 * (2 * odd + (j >> 5)));
      const uint32_t c0 = (l & 0xF) | ((h & 3) << 4), c1 = ((l >> 8) & 0xF) | (((h >> 8) & 3) << 4);
      const int scv = (int)__ldg(sc + 2 * (j >> 5) + ((j & 31) >> 4));
      const __half2 s2 = __half2half2(__int2half_rn(scv));
      out[i] = h2_as_u32(hmul2_rn(d2, hmul2_rn(s2, __hsub2(ints_plus_1024(c0, c1), off))));
    }
  }
  static __device__ __forceinline__ void corr(const uint8_t*, int, int64_t, uint32_t (&)[32]) {}
};

// IQ4_XS: fp32 d*(ls-32)*level rounded once to ab_t, dequantize_block_iq4_xs (dequantize.cuh:420-435)
template <typename ab_t> struct Decoder<T_IQ4_XS, ab_t> {
  static __device__ __forceinline__ void slab(const uint8_t* row, int s, int64_t, const DecodeCtx& cx, uint32_t (&out)[32]) {
    const uint8_t* blk = row + (int64_t)(s >> 2) * 136;
    const uint2 hdr = __ldg(reinterpret_cast<const uint2*>(blk));
    const float d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xffff)));
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      const int ib = 2 * (s & 3) + t;
      const int ls = (int)(((hdr.y >> (4 * ib)) & 0xF) | ((((hdr.x >> 16) >> (2 * ib)) & 3) << 4)) - 32;
      const float dl = d * (float)ls;
      const uint2* qp = reinterpret_cast<const uint2*>(blk + 8 + 16 * ib);
      const uint2 qa = __ldg(qp), qb = __ldg(qp + 1);
      const uint32_t q[4] = {qa.x, qa.y, qb.x, qb.y};
#pragma unroll
      for (int i = 0; i < 4; ++i) {  // bytes 4i..4i+3: values 4i.. (low) and 16+4i.. (high)
        const uint32_t w = q[i];
        out[16 * t + 2 * i] = pack2<ab_t>(dl * (float)cx.kv[w & 0xF], dl * (float)cx.kv[(w >> 8) & 0xF]);
        out[16 * t + 2 * i + 1] = pack2<ab_t>(dl * (float)cx.kv[(w >> 16) & 0xF], dl * (float)cx.kv[(w >> 24) & 0xF]);
        out[16 * t + 8 + 2 * i] = pack2<ab_t>(dl * (float)cx.kv[(w >> 4) & 0xF], dl * (float)cx.kv[(w >> 12) & 0xF]);
        out[16 * t + 8 + 2 * i + 1] = pack2<ab_t>(dl * (float)cx.kv[(w >> 20) & 0xF], dl * (float)cx.kv[(w >> 28) & 0xF]);
      }
    }
  }
  static __device__ __forceinline__ void corr(const uint8_t*, int, int64_t, uint32_t (&)[32]) {}
};

// IQ2_XXS: fp32 d*(0.5+s)*0.25*grid*sign rounded once, dequantize_block_iq2_xxs (dequantize.cuh:258-275)
template <typename ab_t> struct Decoder<T_IQ2_XXS, ab_t> {
  static __device__ __forceinline__ void slab(const uint8_t* row, int s, int64_t, const DecodeCtx& cx, uint32_t (&out)[32]) {
    const uint8_t* blk = row + (int64_t)(s >> 2) * 66;
    const float dh = __half2float(__ushort_as_half((unsigned short)ldg16(blk)));
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      const uint8_t* q2 = blk + 2 + 8 * (2 * (s & 3) + t);
      const uint32_t idx = ldg16(q2) | (ldg16(q2 + 2) << 16);
      const uint32_t aux = ldg16(q2 + 4) | (ldg16(q2 + 6) << 16);
      const float d = dh * (0.5f + (float)(aux >> 28)) * 0.25f;
#pragma unroll
      for (int il = 0; il < 4; ++il) {
        const uint64_t g = cx.grid[(idx >> (8 * il)) & 0xFF];
        const uint32_t sg = cx.signs[(aux >> (7 * il)) & 127];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float a = d * (float)((uint32_t)(g >> (16 * j)) & 0xFF) * ((sg >> (2 * j)) & 1 ? -1.f : 1.f);
          const float b = d * (float)((uint32_t)(g >> (16 * j + 8)) & 0xFF) * ((sg >> (2 * j + 1)) & 1 ? -1.f : 1.f);
          out[16 * t + 4 * il + j] = pack2<ab_t>(a, b);
        }
      }
    }
  }
  static __device__ __forceinline__ void corr(const uint8_t*, int, int64_t, uint32_t (&)[32]) {}
};

// ---- kernel -----------------------------------------------------------------------------

struct MmqParams {
  const uint8_t* w;
  void* y;
  int64_t M, N, K, kpad;
  int nmain, ncorr;           // K slabs of weights / of correction columns
  int64_t row_bytes;
  // MoE
  const int32_t* sorted_ids;
  const int32_t* expert_ids;
  const int32_t* n_post_pad;
  int64_t expert_stride_bytes, rows_out;
  int* status;
};

template <int TYPE, typename ab_t, typename out_t, int TN, bool MOE>
__global__ void __launch_bounds__(MMQ_THREADS, 1) mmq_kernel(const __grid_constant__ CUtensorMap bmap, const MmqParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // carve: the swizzled tiles need 1024-byte alignment
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int B_STAGE = TN * MMQ_BK * 2;
  uint8_t* sA = smem;
  uint8_t* sB = smem + MMQ_STAGES * MMQ_A_STAGE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sB + MMQ_STAGES * B_STAGE);
  uint64_t* full_a = bars;
  uint64_t* full_b = bars + MMQ_STAGES;
  uint64_t* empty = bars + 2 * MMQ_STAGES;
  uint64_t* accum = bars + 3 * MMQ_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * MMQ_STAGES + 1);
  uint64_t* s_grid = reinterpret_cast<uint64_t*>(bars + 3 * MMQ_STAGES + 2);
  uint8_t* s_signs = reinterpret_cast<uint8_t*>(s_grid + 256);
  int8_t* s_kv = reinterpret_cast<int8_t*>(s_signs + 128);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t n0 = (int64_t)blockIdx.x * MMQ_ROWS;
  const int64_t t0 = (int64_t)blockIdx.y * TN;
  const uint8_t* wbase = p.w;
  if (MOE) {
    const int e = p.expert_ids[blockIdx.y];
    if (e < 0 || e > 255) return;                    // same guard as the reference (moe.cuh:33)
    if (t0 >= (int64_t)p.n_post_pad[0]) return;      // nothing routed to this block
    wbase += (int64_t)e * p.expert_stride_bytes;
  }
  constexpr uint32_t TMEM_COLS = TN < 32 ? 32 : TN;
  const int nk = p.nmain + p.ncorr;

  if (threadIdx.x == 0) {
    for (int s = 0; s < MMQ_STAGES; ++s) {
      mbar_init(&full_a[s], 4);
      mbar_init(&full_b[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(accum, 1);
    fence_barrier_init();
  }
  if (TYPE == T_IQ2_XXS) {
    for (int i = threadIdx.x; i < 256; i += blockDim.x) s_grid[i] = d_iq2xxs_grid[i];
    for (int i = threadIdx.x; i < 128; i += blockDim.x) s_signs[i] = d_ksigns_iq2xs[i];
  }
  if (TYPE == T_IQ4_XS && threadIdx.x < 16) s_kv[threadIdx.x] = d_kvalues_iq4nl[threadIdx.x];
  if (warp == 4) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  bool ok = true;

  if (warp < 4) {
    // ---------------- A producers: thread r decodes row n0 + r ----------------
    const int r = threadIdx.x;
    const int64_t n = n0 + r;
    const bool live = n < p.N;
    const uint8_t* row = wbase + (live ? n : 0) * p.row_bytes;
    DecodeCtx cx{s_grid, s_signs, s_kv};
    const uint32_t row_off = (uint32_t)((r >> 3) * 1024 + (r & 7) * 128);
    for (int i = 0; i < nk && ok; ++i) {
      const int s = i % MMQ_STAGES;
      const uint32_t round = (uint32_t)(i / MMQ_STAGES);
      uint32_t v[32];
      if (!live) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = 0;
      } else if (i < p.nmain) {
        Decoder<TYPE, ab_t>::slab(row, i, p.K, cx, v);
      } else {
        Decoder<TYPE, ab_t>::corr(row, i - p.nmain, p.K, v);
      }
      ok = mbar_wait_bounded(&empty[s], (round & 1u) ^ 1u);
      if (!ok) break;
      uint8_t* dst = sA + (size_t)s * MMQ_A_STAGE + row_off;
#pragma unroll
      for (int c = 0; c < 8; ++c)
        *reinterpret_cast<uint4*>(dst + ((c ^ (r & 7)) << 4)) = make_uint4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(&full_a[s]);
    }
    // ---------------- epilogue: TMEM lane r = weight row n0 + r ----------------
    if (ok) ok = mbar_wait_bounded(accum, 0);
    if (ok) {
      tc_fence_after();
      out_t* y = static_cast<out_t*>(p.y);
      const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
      const int64_t npp = MOE ? (int64_t)p.n_post_pad[0] : 0;
#pragma unroll 1
      for (int c0 = 0; c0 < TN; c0 += 16) {
        uint32_t acc[16];
        tmem_ld16(lane_addr + (uint32_t)c0, acc);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int64_t t = t0 + c0 + j;
          int64_t orow;
          if (MOE) {
            orow = (t < npp) ? (int64_t)p.sorted_ids[t] : p.rows_out;
          } else {
            orow = t < p.M ? t : p.rows_out;
          }
          if (live && orow < p.rows_out) y[orow * p.N + n] = from_float<out_t>(__uint_as_float(acc[j]));
        }
      }
    }
  } else if (warp == 4) {
    // ---------------- B loader: one TMA box (64 k x TN rows) per stage ----------------
    if (lane == 0) {
      for (int i = 0; i < nk; ++i) {
        const int s = i % MMQ_STAGES;
        const uint32_t round = (uint32_t)(i / MMQ_STAGES);
        if (!mbar_wait_bounded(&empty[s], (round & 1u) ^ 1u)) { ok = false; break; }
        const int64_t col = i < p.nmain ? (int64_t)i * MMQ_BK : p.kpad + (int64_t)(i - p.nmain) * MMQ_BK;
        mbar_expect_tx(&full_b[s], (uint32_t)B_STAGE);
        tma_load_2d(sB + (size_t)s * B_STAGE, &bmap, (int)col, (int)t0, &full_b[s]);
      }
    }
  } else {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(MMQ_ROWS, TN, sizeof(ab_t) == 2 && std::is_same<ab_t, __nv_bfloat16>::value ? 1 : 0);
      for (int i = 0; i < nk; ++i) {
        const int s = i % MMQ_STAGES;
        const uint32_t round = (uint32_t)(i / MMQ_STAGES);
        if (!mbar_wait_bounded(&full_a[s], round & 1u) || !mbar_wait_bounded(&full_b[s], round & 1u)) { ok = false; break; }
        tc_fence_after();
        const uint64_t ad = umma_desc_sw128(smem_u32(sA + (size_t)s * MMQ_A_STAGE));
        const uint64_t bd = umma_desc_sw128(smem_u32(sB + (size_t)s * B_STAGE));
#pragma unroll
        for (int kk = 0; kk < MMQ_BK / 16; ++kk)  // 16 values = 32 bytes = +2 in the descriptor's 16-byte units
          umma_f16(tmem_base, ad + 2 * kk, bd + 2 * kk, idesc, (i > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&empty[s]);
      }
      if (ok) umma_commit(accum);
    }
  }
  if (!ok && lane == 0) atomicExch(p.status, E_TIMEOUT);
  tc_fence_before();
  __syncthreads();
  if (warp == 4) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ---- host side --------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

int mmq_moe_block_size() { return 64; }

static int pick_tn(int64_t M) {
  if (M <= 16) return 16;
  if (M <= 32) return 32;
  if (M <= 64) return 64;
  if (M <= 128) return 128;
  return 256;
}

template <int TYPE, typename ab_t, typename out_t, int TN, bool MOE>
static int launch_tn(const MmqArgs& a, const MmqParams& p, int64_t b_rows, cudaStream_t stream) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return E_CUDA;
  CUtensorMap map;
  const cuuint64_t dims[2] = {(cuuint64_t)a.ldb, (cuuint64_t)b_rows};
  const cuuint64_t strides[1] = {(cuuint64_t)a.ldb * 2};
  const cuuint32_t box[2] = {MMQ_BK, (cuuint32_t)TN};
  const cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = std::is_same<ab_t, __nv_bfloat16>::value ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  if (enc(&map, dt, 2, const_cast<void*>(a.b), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return E_CUDA;
  auto kern = mmq_kernel<TYPE, ab_t, out_t, TN, MOE>;
  const size_t smem = 1024 + (size_t)MMQ_STAGES * (MMQ_A_STAGE + TN * MMQ_BK * 2) + (3 * MMQ_STAGES + 2) * 8 + 2048 + 128 + 16;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return E_CUDA;
    configured[dev & 63] = true;
  }
  dim3 grid((unsigned)((a.N + MMQ_ROWS - 1) / MMQ_ROWS), (unsigned)((b_rows + TN - 1) / TN), 1);
  kern<<<grid, MMQ_THREADS, smem, stream>>>(map, p);
  return cudaGetLastError() == cudaSuccess ? E_OK : E_CUDA;
}

template <int TYPE, typename ab_t, typename out_t>
static int launch_shape(const MmqArgs& a, const MmqParams& p, cudaStream_t s) {
  if (a.sorted_ids) return launch_tn<TYPE, ab_t, out_t, 64, true>(a, p, a.n_sorted, s);
  switch (pick_tn(a.M)) {
    case 16: return launch_tn<TYPE, ab_t, out_t, 16, false>(a, p, a.M, s);
    case 32: return launch_tn<TYPE, ab_t, out_t, 32, false>(a, p, a.M, s);
    case 64: return launch_tn<TYPE, ab_t, out_t, 64, false>(a, p, a.M, s);
    case 128: return launch_tn<TYPE, ab_t, out_t, 128, false>(a, p, a.M, s);
    default: return launch_tn<TYPE, ab_t, out_t, 256, false>(a, p, a.M, s);
  }
}

template <int TYPE, typename ab_t>
static int launch_out(const MmqArgs& a, const MmqParams& p, cudaStream_t s) {
  switch (a.out_dtype) {
    case DT_F32: return launch_shape<TYPE, ab_t, float>(a, p, s);
    case DT_F16: return launch_shape<TYPE, ab_t, __half>(a, p, s);
    case DT_BF16: return launch_shape<TYPE, ab_t, __nv_bfloat16>(a, p, s);
  }
  return E_BAD_DTYPE;
}

int launch_mmq(const MmqArgs& a, cudaStream_t stream) {
  if (a.N == 0 || a.M == 0) return E_OK;
  MmqParams p{};
  p.w = static_cast<const uint8_t*>(a.w);
  p.y = a.y;
  p.M = a.M;
  p.N = a.N;
  p.K = a.K;
  p.kpad = round_up(a.K, 512);
  p.nmain = (int)((a.K + MMQ_BK - 1) / MMQ_BK);
  p.ncorr = a.corr_mode == CORR_NONE ? 0 : (int)((a.K / 32 + MMQ_BK - 1) / MMQ_BK);
  p.row_bytes = a.K / block_size(a.type) * type_size(a.type);
  p.sorted_ids = a.sorted_ids;
  p.expert_ids = a.expert_ids;
  p.n_post_pad = a.n_post_pad;
  p.expert_stride_bytes = a.expert_stride_bytes;
  p.rows_out = a.rows_out;
  p.status = a.status;
  const bool bf = a.b_dtype == DT_BF16;
  switch (a.type) {
    case T_Q4_0: return bf ? E_BAD_DTYPE : launch_out<T_Q4_0, __half>(a, p, stream);
    case T_Q8_0: return bf ? E_BAD_DTYPE : launch_out<T_Q8_0, __half>(a, p, stream);
    case T_Q4_K: return bf ? E_BAD_DTYPE : launch_out<T_Q4_K, __half>(a, p, stream);
    case T_Q6_K: return bf ? E_BAD_DTYPE : launch_out<T_Q6_K, __half>(a, p, stream);
    case T_IQ2_XXS: return bf ? launch_out<T_IQ2_XXS, __nv_bfloat16>(a, p, stream) : launch_out<T_IQ2_XXS, __half>(a, p, stream);
    case T_IQ4_XS: return bf ? launch_out<T_IQ4_XS, __nv_bfloat16>(a, p, stream) : launch_out<T_IQ4_XS, __half>(a, p, stream);
  }
  return E_BAD_TYPE;
}

}  // namespace gguf_b200
