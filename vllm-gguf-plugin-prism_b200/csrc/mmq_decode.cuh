// Weight decoders of the tensor-core GEMM (mmq.cu): one 32-value group of one weight row
// ("unit" u = values 32u..32u+31) -> 16 packed 16-bit pairs = 64 bytes of the row in the A tile.
// A producer thread owns one row of a 64-value stage and calls a decoder for its two units
// (the whole-stage decoders at the end of this file replace that for Q4_K / Q4_0 / Q8_0).
//
// Each decoder is split in two:
//   load()   fetches a unit's raw bytes (from the shared-memory raw ring) into registers,
//   decode() turns those registers into fp16/bf16 values.
//
// Values are bit-identical to the reference's standalone dequantize for the types that are fed
// to the MMA as dequantized weights (Q4_0, Q8_0, Q6_K: dequantize.cuh:3-15, 69-78, 232-256;
// IQ4_XS, IQ2_XXS: dequantize.cuh:420-435, 258-275).  Q4_K feeds half(d*sc*q) and carries its
// min term in the correction columns (see mmq.cu).
//
// Blocks of Q4_0 / Q8_0 / Q6_K / IQ2_XXS are only 2-byte aligned: raw bytes are fetched as the
// aligned 32-bit words that cover them and realigned with funnel shifts.
#pragma once

#include "common.cuh"

namespace gguf_b200 {

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

// N aligned words covering `len` bytes from the (2-byte aligned) address p in the shared-memory
// staging area of the raw weight bytes; words that hold no needed byte are not loaded.  The loads
// are explicit shared-window loads: rounding the address down through an integer made the
// compiler forget the address space, and generic loads of shared memory travel the global-memory
// pipeline (ncu: `lg_throttle` and `long_scoreboard` stalls in the decode warps).
template <int N> __device__ __forceinline__ void ldg_cover(const uint8_t* p, int len, uint32_t* r) {
  const uint32_t a = smem_u32(p);
  const uint32_t al = a & ~3u;
  const int need = (len + (int)(a & 3u) + 3) >> 2;
#pragma unroll
  for (int i = 0; i < N; ++i) r[i] = i < need ? lds32(al + 4u * i) : 0u;
}
// word i of the byte stream that starts `sh` bits into r[0]
__device__ __forceinline__ uint32_t word_at(const uint32_t* r, int i, uint32_t sh) { return __funnelshift_r(r[i], r[i + 1], sh); }
__device__ __forceinline__ uint32_t shift_of(const uint8_t* p) { return (uint32_t)(reinterpret_cast<uintptr_t>(p) & 3) * 8u; }

// Tables in shared memory, held as 32-bit shared-window addresses so that every look-up is an
// ld.shared (through a generic pointer the look-ups travel the global-memory pipeline).  The
// look-ups are plain (non-volatile) asm: their index comes from weight bytes that are read long
// after the barrier that published the tables.
struct DecodeCtx {
  // The two IQ2_XXS tables are replicated, entry i of copy c at index COPIES * i + c -- the sign table
  // (16-byte entries) eight times, the selector table (8-byte entries) sixteen times -- and a thread
  // reads copy (lane mod COPIES): the lanes that share a 128-byte access phase then sit in different
  // columns of the 128 bytes whatever entries they look up (random look-ups into a single copy averaged
  // 2.5 to 3 bank conflicts per access).  `sel` and `sgn` already point at this thread's copy.
  uint32_t sel;       // IQ2_XXS: per grid entry (8 bytes), the byte-permute selectors of its four value pairs (see Decoder<T_IQ2_XXS>)
  uint32_t sgn;       // IQ2_XXS: per 7-bit sign index (16 bytes), the sign-bit masks of the four value pairs
  uint32_t kv;        // IQ4_NL / IQ4_XS: the 16 levels, one signed byte each
  __device__ __forceinline__ uint2 sel_at(uint32_t i) const {
    uint2 v;
    asm("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(sel + 128u * i));
    return v;
  }
  __device__ __forceinline__ uint4 sgn_at(uint32_t i) const {
    uint4 v;
    asm("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(sgn + 128u * i));
    return v;
  }
  __device__ __forceinline__ float level(uint32_t i) const {
    int v;
    asm("ld.shared.s8 %0, [%1];" : "=r"(v) : "r"(kv + i));
    return (float)v;
  }
};
// Shared-memory tables of the IQ2_XXS decoder, built once per CTA from the format's grid and
// sign tables.  A grid entry holds eight magnitudes, each one of {8, 25, 43}; with the three
// products d*8, d*25, d*43 of a 32-value group rounded to 16 bits and parked in two registers,
// every PAIR of decoded values is one byte-permute whose 16-bit selector depends only on the grid
// entry -- those selectors are what the table holds -- and the signs are one XOR per pair.
__device__ __forceinline__ uint2 iq2xxs_pair_selectors(uint64_t grid_entry) {
  uint32_t s[2] = {0u, 0u};
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint32_t m = (uint32_t)(grid_entry >> (8 * j)) & 0xFFu;
    const uint32_t c = (m > 8u ? 1u : 0u) + (m > 25u ? 1u : 0u);   // which of the three magnitudes
    const uint32_t nib = (2u * c) | ((2u * c + 1u) << 4);           // its two bytes in the register pair
    s[j >> 2] |= nib << (8 * (j & 3));
  }
  return make_uint2(s[0], s[1]);
}
__device__ __forceinline__ uint4 iq2xxs_pair_signs(uint32_t sign_bits) {
  uint32_t m[4];
#pragma unroll
  for (int p = 0; p < 4; ++p) m[p] = (((sign_bits >> (2 * p)) & 1u) << 15) | (((sign_bits >> (2 * p + 1)) & 1u) << 31);
  return make_uint4(m[0], m[1], m[2], m[3]);
}

template <int TYPE, typename ab_t> struct Decoder;

// Raw-byte staging of the tensor-core kernel: KC values of every row of the tile are copied to
// shared memory at once (coalesced 16-byte pieces), RBC bytes per row, in slots of SLOT bytes.
// SLOT leaves room for the 16-byte rounding of the start and is an odd multiple of 16 so that
// the 128 rows of a tile spread over all shared-memory banks.
// TMA variant of the staging (row bytes a multiple of 16 and chunk starts 16-byte aligned): a
// chunk of KC_T values per row is one 2-D box of RBC_T bytes x 128 rows, stored densely.  RBC_T
// is an odd multiple of 16 for every supported type, so dense rows are bank-conflict free as well.
template <int TYPE> struct TmaGeom {
  static constexpr bool OK = TYPE == T_Q4_0 || TYPE == T_Q8_0 || TYPE == T_Q4_K || TYPE == T_Q5_K || TYPE == T_IQ4_XS;
  static constexpr int KC_T = TYPE == T_IQ4_XS ? 512 : 256;
  static constexpr int RBC_T = KC_T / BlockTraits<TYPE>::QK * BlockTraits<TYPE>::TS;   // 144, 176 or 272
};
template <int TYPE> struct RawGeom {
  static constexpr int KC = TYPE == T_IQ2_XXS ? 512 : 256;   // multiples of 256: every producer group meets every chunk
  static constexpr int RBC = KC / BlockTraits<TYPE>::QK * BlockTraits<TYPE>::TS;
  static constexpr int S16 = (RBC + 30) / 16 + 1;
  static constexpr int SLOT = (S16 % 2 ? S16 : S16 + 1) * 16;
};

// Types whose two 32-value units of a 64-value stage (units 2j and 2j + 1 of a 256-value super-block, always
// whole) are cut from the same words of the block: load() depends on the unit only through u >> 1.
template <int TYPE> __host__ __device__ constexpr bool decoder_pair_load() { return TYPE == T_Q2_K || TYPE == T_Q3_K || TYPE == T_Q5_K || TYPE == T_Q6_K; }

// ---- Q4_0: value = half(q * d), q unsigned (see Stage64<T_Q4_0>); unit = one 18-byte block ----
template <typename ab_t> struct Decoder<T_Q4_0, ab_t> {
  static constexpr int CORR_OFF = 0;   // byte offset in a block of the fp16 that is the block's correction value (-1: none / computed)
  static constexpr int RW = 7;   // 18 bytes at 2-byte alignment: <= 6 words (+1 for the shifts)
  static __device__ __forceinline__ void load(const uint8_t* row, int u, uint32_t (&raw)[RW]) {
    ldg_cover<RW - 1>(row + (int64_t)u * 18, 18, raw);
    raw[RW - 1] = 0;
  }
  static __device__ __forceinline__ void decode(const uint8_t* row, int u, const uint32_t (&raw)[RW], const DecodeCtx&, uint32_t (&out)[16]) {
    const uint32_t sh = shift_of(row + (int64_t)u * 18);
    const __half2 off = __floats2half2_rn(1024.f, 1024.f);
    const uint32_t du = word_at(raw, 0, sh) & 0xFFFFu;
    const __half2 d2 = u32_as_h2(du | (du << 16));
#pragma unroll
    for (int i = 0; i < 8; ++i) {  // stream half-word 1+i holds qs[2i], qs[2i+1]
      const int h = 1 + i;
      const uint32_t wv = word_at(raw, h >> 1, sh);
      const uint32_t t = (h & 1) ? (wv >> 16) : (wv & 0xFFFFu);
      out[i] = h2_as_u32(hmul2_rn(__hsub2(ints_plus_1024(t & 0xF, (t >> 8) & 0xF), off), d2));
      out[8 + i] = h2_as_u32(hmul2_rn(__hsub2(ints_plus_1024((t >> 4) & 0xF, (t >> 12) & 0xF), off), d2));
    }
  }
  // correction columns [32c, 32c+32): A'[n, g] = d of block g (pairs with -8 * s8 on the B side)
  static __device__ __forceinline__ void corr(const uint8_t* row, int c, int64_t K, uint32_t (&out)[16]) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int64_t g = 32 * (int64_t)c + 2 * i;
      const uint32_t a = g * 32 < K ? ldg16(row + g * 18) : 0u;
      const uint32_t b = (g + 1) * 32 < K ? ldg16(row + (g + 1) * 18) : 0u;
      out[i] = a | (b << 16);
    }
  }
};

// ---- Q8_0: value = half(q * d); unit = one 34-byte block ---------------------------------------
template <typename ab_t> struct Decoder<T_Q8_0, ab_t> {
  static constexpr int CORR_OFF = -1;   // byte offset in a block of the fp16 that is the block's correction value (-1: none / computed)
  static constexpr int RW = 11;  // 34 bytes: <= 10 words (+1)
  static __device__ __forceinline__ void load(const uint8_t* row, int u, uint32_t (&raw)[RW]) {
    ldg_cover<RW - 1>(row + (int64_t)u * 34, 34, raw);
    raw[RW - 1] = 0;
  }
  static __device__ __forceinline__ void decode(const uint8_t* row, int u, const uint32_t (&raw)[RW], const DecodeCtx&, uint32_t (&out)[16]) {
    const uint32_t sh = shift_of(row + (int64_t)u * 34);
    const __half2 off = __floats2half2_rn(1152.f, 1152.f);  // 1024 + 128
    const uint32_t du = word_at(raw, 0, sh) & 0xFFFFu;
    const __half2 d2 = u32_as_h2(du | (du << 16));
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int h = 1 + i;
      const uint32_t wv = word_at(raw, h >> 1, sh);
      const uint32_t t = ((h & 1) ? (wv >> 16) : (wv & 0xFFFFu)) ^ 0x8080u;  // int8 -> biased unsigned
      out[i] = h2_as_u32(hmul2_rn(__hsub2(ints_plus_1024(t & 0xFF, t >> 8), off), d2));
    }
  }
  static __device__ __forceinline__ void corr(const uint8_t*, int, int64_t, uint32_t (&)[16]) {}
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

// ---- Q4_K: A = half(d1 * q) with d1 = half(d * sc); the -dmin*m part is a correction column ----
// unit u: super-block u>>3, sub-block j = u&7: nibble (j&1) of the 32 bytes qs[32*(j>>1) ..]
template <typename ab_t> struct Decoder<T_Q4_K, ab_t> {
  static constexpr int CORR_OFF = -1;   // byte offset in a block of the fp16 that is the block's correction value (-1: none / computed)
  static constexpr int RW = 12;  // header (16 bytes) + 32 bytes of nibbles, all 16-byte aligned
  static __device__ __forceinline__ void load(const uint8_t* row, int u, uint32_t (&raw)[RW]) {
    const uint8_t* blk = row + (int64_t)(u >> 3) * 144;
    const uint32_t sb = smem_u32(blk), sq = sb + 16 + 32 * ((u >> 1) & 3);
    const uint4 h = lds128s(sb), a = lds128s(sq), b = lds128s(sq + 16);
    raw[0] = h.x; raw[1] = h.y; raw[2] = h.z; raw[3] = h.w;
    raw[4] = a.x; raw[5] = a.y; raw[6] = a.z; raw[7] = a.w; raw[8] = b.x; raw[9] = b.y; raw[10] = b.z; raw[11] = b.w;
  }
  static __device__ __forceinline__ void decode(const uint8_t*, int u, const uint32_t (&raw)[RW], const DecodeCtx&, uint32_t (&out)[16]) {
    const int j = u & 7, sh = 4 * (j & 1);
    const __half dall = __ushort_as_half((unsigned short)(raw[0] & 0xffff));
    int sc, m;
    q4k_scale_min(raw[1], raw[2], raw[3], j, sc, m);
    (void)m;
    const __half2 dv = __half2half2(__hmul_rn(dall, __int2half_rn(sc)));
    const __half2 off = __floats2half2_rn(1024.f, 1024.f);
#pragma unroll
    for (int i = 0; i < 8; ++i) {  // word i: bytes 4i..4i+3 -> values 4i..4i+3 of this sub-block
      const uint32_t w = raw[4 + i] >> sh;
      out[2 * i] = h2_as_u32(hmul2_rn(__hsub2(ints_plus_1024(w & 0xF, (w >> 8) & 0xF), off), dv));
      out[2 * i + 1] = h2_as_u32(hmul2_rn(__hsub2(ints_plus_1024((w >> 16) & 0xF, (w >> 24) & 0xF), off), dv));
    }
  }
  // correction columns [32c, 32c+32): A'[n, g] = half(dmin * m_g)  (pairs with -s8 on the B side)
  static __device__ __forceinline__ void corr(const uint8_t* row, int c, int64_t K, uint32_t (&out)[16]) {
#pragma unroll
    for (int sb = 0; sb < 4; ++sb) {
      const int64_t sbi = 4 * (int64_t)c + sb;  // super-block index: 8 groups each
      if (sbi * 256 >= K) {
#pragma unroll
        for (int i = 0; i < 4; ++i) out[4 * sb + i] = 0;
        continue;
      }
      const uint4 hdr = __ldg(reinterpret_cast<const uint4*>(row + sbi * 144));
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

// ---- Q4_1: A = half(q * d); the min term m * s8 is a correction column (B side: +s8) -----------------
template <typename ab_t> struct Decoder<T_Q4_1, ab_t> {
  static constexpr int CORR_OFF = 2;   // byte offset in a block of the fp16 that is the block's correction value (-1: none / computed)
  static constexpr int RW = 5;   // 20 bytes, 4-byte aligned
  static __device__ __forceinline__ void load(const uint8_t* row, int u, uint32_t (&raw)[RW]) {
    const uint32_t sb = smem_u32(row + (int64_t)u * 20);
#pragma unroll
    for (int i = 0; i < 5; ++i) raw[i] = lds32(sb + 4u * i);
  }
  static __device__ __forceinline__ void decode(const uint8_t*, int, const uint32_t (&raw)[RW], const DecodeCtx&, uint32_t (&out)[16]) {
    const uint32_t du = raw[0] & 0xFFFFu;
    const __half2 d2 = u32_as_h2(du | (du << 16)), off = __floats2half2_rn(1024.f, 1024.f);
#pragma unroll
    for (int k = 0; k < 4; ++k) {  // word k = qs[4k..4k+3]: values 4k.. (low nibbles) and 16 + 4k.. (high); halves 1024 + code by byte-permute
      const uint32_t cl = raw[1 + k] & 0x0F0F0F0Fu, ch = (raw[1 + k] >> 4) & 0x0F0F0F0Fu;
      out[2 * k] = h2_as_u32(hmul2_rn(__hsub2(u32_as_h2(__byte_perm(cl, 0x64646464u, 0x4140)), off), d2));
      out[2 * k + 1] = h2_as_u32(hmul2_rn(__hsub2(u32_as_h2(__byte_perm(cl, 0x64646464u, 0x4342)), off), d2));
      out[8 + 2 * k] = h2_as_u32(hmul2_rn(__hsub2(u32_as_h2(__byte_perm(ch, 0x64646464u, 0x4140)), off), d2));
      out[8 + 2 * k + 1] = h2_as_u32(hmul2_rn(__hsub2(u32_as_h2(__byte_perm(ch, 0x64646464u, 0x4342)), off), d2));
    }
  }
  // correction columns [32c, 32c+32): A'[n, g] = m of block g
  static __device__ __forceinline__ void corr(const uint8_t* row, int c, int64_t K, uint32_t (&out)[16]) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int64_t g = 32 * (int64_t)c + 2 * i;
      const uint32_t a = g * 32 < K ? ldg16(row + g * 20 + 2) : 0u;
      const uint32_t b = (g + 1) * 32 < K ? ldg16(row + (g + 1) * 20 + 2) : 0u;
      out[i] = a | (b << 16);
    }
  }
};

// fifth bits: bit j of qh belongs to value j
// Word k of a 5-bit legacy block (qs[4k..4k+3]) -> the four pairs it holds: values 4k, 4k+1 | 4k+2, 4k+3 (low nibbles,
// fifth bits 4k.. of qh) and 16+4k.. (high nibbles, fifth bits 16+4k..).  Four consecutive bits of qh are spread to bit 4
// of four bytes with one multiplication (t * 0x02040810 puts bit j of t at bit 8j + 4, no carries for t < 16), the code
// bytes become halves 1024 + code by byte-permute, the offset is subtracted exactly and d multiplies once.
__device__ __forceinline__ void q5_word(uint32_t q, uint32_t qh, int k, __half2 off, __half2 d2, uint32_t& lo01, uint32_t& lo23,
                                        uint32_t& hi01, uint32_t& hi23) {
  const uint32_t cl = (q & 0x0F0F0F0Fu) | ((((qh >> (4 * k)) & 0xFu) * 0x02040810u) & 0x10101010u);
  const uint32_t ch = ((q >> 4) & 0x0F0F0F0Fu) | ((((qh >> (16 + 4 * k)) & 0xFu) * 0x02040810u) & 0x10101010u);
  lo01 = h2_as_u32(hmul2_rn(__hsub2(u32_as_h2(__byte_perm(cl, 0x64646464u, 0x4140)), off), d2));
  lo23 = h2_as_u32(hmul2_rn(__hsub2(u32_as_h2(__byte_perm(cl, 0x64646464u, 0x4342)), off), d2));
  hi01 = h2_as_u32(hmul2_rn(__hsub2(u32_as_h2(__byte_perm(ch, 0x64646464u, 0x4140)), off), d2));
  hi23 = h2_as_u32(hmul2_rn(__hsub2(u32_as_h2(__byte_perm(ch, 0x64646464u, 0x4342)), off), d2));
}

// ---- Q5_0: value = half((q - 16) * d), 22-byte blocks (2-byte aligned): d | qh[4] | qs[16] ------------
template <typename ab_t> struct Decoder<T_Q5_0, ab_t> {
  static constexpr int CORR_OFF = -1;   // byte offset in a block of the fp16 that is the block's correction value (-1: none / computed)
  static constexpr int RW = 8;   // 22 bytes at 2-byte alignment: <= 6 words (+ shifts)
  static __device__ __forceinline__ void load(const uint8_t* row, int u, uint32_t (&raw)[RW]) {
    ldg_cover<7>(row + (int64_t)u * 22, 22, raw);
    raw[7] = 0;
  }
  static __device__ __forceinline__ void decode(const uint8_t* row, int u, const uint32_t (&raw)[RW], const DecodeCtx&, uint32_t (&out)[16]) {
    const uint32_t sh = shift_of(row + (int64_t)u * 22);
    const uint32_t w0 = word_at(raw, 0, sh), w1 = word_at(raw, 1, sh);
    const uint32_t du = w0 & 0xFFFFu, qh = (w0 >> 16) | (w1 << 16);
    const __half2 d2 = u32_as_h2(du | (du << 16)), off = __floats2half2_rn(1040.f, 1040.f);   // 1024 + 16
#pragma unroll
    for (int k = 0; k < 4; ++k) {  // bytes 6 + 4k .. of the block = qs[4k..4k+3]: values 4k.. (low nibbles) and 16 + 4k.. (high)
      const uint32_t q = __funnelshift_r(word_at(raw, 1 + k, sh), word_at(raw, 2 + k, sh), 16);
      q5_word(q, qh, k, off, d2, out[2 * k], out[2 * k + 1], out[8 + 2 * k], out[8 + 2 * k + 1]);
    }
  }
  static __device__ __forceinline__ void corr(const uint8_t*, int, int64_t, uint32_t (&)[16]) {}
};

// ---- Q5_1: A = half(q * d), 24-byte blocks (8-byte aligned): d | m | qh[4] | qs[16]; correction column m ----
template <typename ab_t> struct Decoder<T_Q5_1, ab_t> {
  static constexpr int CORR_OFF = 2;   // byte offset in a block of the fp16 that is the block's correction value (-1: none / computed)
  static constexpr int RW = 6;
  static __device__ __forceinline__ void load(const uint8_t* row, int u, uint32_t (&raw)[RW]) {
    const uint32_t sb = smem_u32(row + (int64_t)u * 24);
    const uint2 a0 = lds64(sb), a1 = lds64(sb + 8), a2 = lds64(sb + 16);
    raw[0] = a0.x; raw[1] = a0.y; raw[2] = a1.x; raw[3] = a1.y; raw[4] = a2.x; raw[5] = a2.y;
  }
  static __device__ __forceinline__ void decode(const uint8_t*, int, const uint32_t (&raw)[RW], const DecodeCtx&, uint32_t (&out)[16]) {
    const uint32_t du = raw[0] & 0xFFFFu, qh = raw[1];
    const __half2 d2 = u32_as_h2(du | (du << 16)), off = __floats2half2_rn(1024.f, 1024.f);
#pragma unroll
    for (int k = 0; k < 4; ++k) q5_word(raw[2 + k], qh, k, off, d2, out[2 * k], out[2 * k + 1], out[8 + 2 * k], out[8 + 2 * k + 1]);
  }
  static __device__ __forceinline__ void corr(const uint8_t* row, int c, int64_t K, uint32_t (&out)[16]) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int64_t g = 32 * (int64_t)c + 2 * i;
      const uint32_t a = g * 32 < K ? ldg16(row + g * 24 + 2) : 0u;
      const uint32_t b = (g + 1) * 32 < K ? ldg16(row + (g + 1) * 24 + 2) : 0u;
      out[i] = a | (b << 16);
    }
  }
};

// ---- Q5_K: A = half(d1 * q), d1 = half(d * sc), q = 4 bits of qs | fifth bit of qh; -dmin*m is a correction column ----
// 176-byte blocks (16-byte aligned): d | dmin | scales[12] | qh[32] | qs[128].  unit u: sub-block j = u&7:
// nibble (j&1) of qs[32*(j>>1) + l], bit j of qh[l], l = 0..31.
template <typename ab_t> struct Decoder<T_Q5_K, ab_t> {
  static constexpr int CORR_OFF = -1;   // byte offset in a block of the fp16 that is the block's correction value (-1: none / computed)
  static constexpr int RW = 20;  // header (16) + 32 bytes of nibbles + 32 bytes of high bits
  static __device__ __forceinline__ void load(const uint8_t* row, int u, uint32_t (&raw)[RW]) {
    const uint8_t* blk = row + (int64_t)(u >> 3) * 176;
    const uint32_t sb = smem_u32(blk), sq = sb + 48 + 32 * ((u >> 1) & 3);
    const uint4 h = lds128s(sb), a = lds128s(sq), b = lds128s(sq + 16), c = lds128s(sb + 16), e = lds128s(sb + 32);
    raw[0] = h.x; raw[1] = h.y; raw[2] = h.z; raw[3] = h.w;
    raw[4] = a.x; raw[5] = a.y; raw[6] = a.z; raw[7] = a.w; raw[8] = b.x; raw[9] = b.y; raw[10] = b.z; raw[11] = b.w;
    raw[12] = c.x; raw[13] = c.y; raw[14] = c.z; raw[15] = c.w; raw[16] = e.x; raw[17] = e.y; raw[18] = e.z; raw[19] = e.w;
  }
  static __device__ __forceinline__ void decode(const uint8_t*, int u, const uint32_t (&raw)[RW], const DecodeCtx&, uint32_t (&out)[16]) {
    const int j = u & 7, sh = 4 * (j & 1);
    const __half dall = __ushort_as_half((unsigned short)(raw[0] & 0xffff));
    int sc, m;
    q4k_scale_min(raw[1], raw[2], raw[3], j, sc, m);
    (void)m;
    const __half2 dv = __half2half2(__hmul_rn(dall, __int2half_rn(sc)));
    const __half2 off = __floats2half2_rn(1024.f, 1024.f);
#pragma unroll
    for (int i = 0; i < 8; ++i) {  // word i: bytes 4i..4i+3 -> values 4i..4i+3 of this sub-block
      const uint32_t w = raw[4 + i] >> sh, hb = (raw[12 + i] >> j) & 0x01010101u;
      const uint32_t c0 = (w & 0xF) | ((hb & 1u) << 4), c1 = ((w >> 8) & 0xF) | (((hb >> 8) & 1u) << 4);
      const uint32_t c2 = ((w >> 16) & 0xF) | (((hb >> 16) & 1u) << 4), c3 = ((w >> 24) & 0xF) | (((hb >> 24) & 1u) << 4);
      out[2 * i] = h2_as_u32(hmul2_rn(__hsub2(ints_plus_1024(c0, c1), off), dv));
      out[2 * i + 1] = h2_as_u32(hmul2_rn(__hsub2(ints_plus_1024(c2, c3), off), dv));
    }
  }
  // correction columns [32c, 32c+32): A'[n, g] = half(dmin * m_g)  (pairs with -s8 on the B side)
  static __device__ __forceinline__ void corr(const uint8_t* row, int c, int64_t K, uint32_t (&out)[16]) {
#pragma unroll
    for (int sb = 0; sb < 4; ++sb) {
      const int64_t sbi = 4 * (int64_t)c + sb;
      if (sbi * 256 >= K) {
#pragma unroll
        for (int i = 0; i < 4; ++i) out[4 * sb + i] = 0;
        continue;
      }
      const uint4 hdr = __ldg(reinterpret_cast<const uint4*>(row + sbi * 176));
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

// ---- Q6_K: value = half(d * half(sc * (code - 32))) ------------------------------------------
// unit u: super-block u>>3, group g = u&7: ip = g>>2 (128-value half), q = g&3:
//   low 4 bits = nibble (q>>1) of ql[64ip + 32(q&1) + l], high 2 bits = bits 2q.. of qh[32ip + l], l = 0..31,
//   scales sc[8ip + 2q] (l < 16) and sc[8ip + 2q + 1].
// The units 2j and 2j + 1 of a stage differ in q & 1 only, so one load serves both (decoder_pair_load):
// Raw: [0..17] the 64 bytes of ql of the half (+ cover), [18..27] 32 bytes of qh (+ cover), [28..30] the four
// scale bytes of the pair (+ cover), [31] d.
template <typename ab_t> struct Decoder<T_Q6_K, ab_t> {
  static constexpr int CORR_OFF = -1;   // byte offset in a block of the fp16 that is the block's correction value (-1: none / computed)
  static constexpr int RW = 32;
  static __device__ __forceinline__ void load(const uint8_t* row, int u, uint32_t (&raw)[RW]) {
    const uint8_t* blk = row + (int64_t)(u >> 3) * 210;
    const int g = u & 7, ip = g >> 2, q = g & 2;
    ldg_cover<17>(blk + 64 * ip, 64, raw);
    raw[17] = 0;
    ldg_cover<9>(blk + 128 + 32 * ip, 32, raw + 18);
    raw[27] = 0;
    ldg_cover<2>(blk + 192 + 8 * ip + 2 * q, 4, raw + 28);
    raw[30] = 0;
    ldg_cover<1>(blk + 208, 2, raw + 31);
  }
  static __device__ __forceinline__ void decode(const uint8_t* row, int u, const uint32_t (&raw)[RW], const DecodeCtx&, uint32_t (&out)[16]) {
    const uint8_t* blk = row + (int64_t)(u >> 3) * 210;
    const int g = u & 7, ip = g >> 2, q = g & 3;
    const uint32_t sh_l = shift_of(blk + 64 * ip), sh_h = shift_of(blk + 128 + 32 * ip);
    const uint32_t sc2 = (word_at(raw + 28, 0, shift_of(blk + 192 + 8 * ip + 2 * (q & 2))) >> (16 * (q & 1))) & 0xFFFFu;   // two int8 scales
    const uint32_t du = (raw[31] >> shift_of(blk + 208)) & 0xFFFFu;
    const __half2 d2 = u32_as_h2(du | (du << 16));
    const __half2 off = __floats2half2_rn(1056.f, 1056.f);  // 1024 + 32
    const __half2 s_lo = __half2half2(__int2half_rn((int)(int8_t)(sc2 & 0xFF)));
    const __half2 s_hi = __half2half2(__int2half_rn((int)(int8_t)(sc2 >> 8)));
    // the 6-bit code of each of a word's four values as one byte: low nibble from ql, bits 4-5 from qh
    // rotated into place; one byte-permute per pair then builds the halves 1024 + code (0x6400 | code)
    const uint32_t sl = 4 * (q >> 1), rot_h = (uint32_t)(2 * q - 4) & 31u;
#pragma unroll
    for (int wi = 0; wi < 8; ++wi) {             // word wi: values 4wi..4wi+3 of the unit
      const uint32_t l = word_at(raw, wi + 8 * (q & 1), sh_l) >> sl;
      const uint32_t h = word_at(raw + 18, wi, sh_h);
      const uint32_t c = (l & 0x0F0F0F0Fu) | (__funnelshift_r(h, h, rot_h) & 0x30303030u);
      const __half2 s2 = wi < 4 ? s_lo : s_hi;
      const __half2 p0 = u32_as_h2(__byte_perm(c, 0x64646464u, 0x4140)), p1 = u32_as_h2(__byte_perm(c, 0x64646464u, 0x4342));
      out[2 * wi] = h2_as_u32(hmul2_rn(d2, hmul2_rn(s2, __hsub2(p0, off))));
      out[2 * wi + 1] = h2_as_u32(hmul2_rn(d2, hmul2_rn(s2, __hsub2(p1, off))));
    }
  }
  static __device__ __forceinline__ void corr(const uint8_t*, int, int64_t, uint32_t (&)[16]) {}
};

// ---- Q2_K: value = fp32 (d*sc)*q - dmin*m rounded once (the dequantized weight itself: the 16-value
// sub-blocks are finer than the 32-value sums of q8_1, so the min term cannot ride in a correction
// column); unit = 32-value group g = u&7 = 4n + j: bytes qs[32n..32n+31] >> 2j, scales 2g, 2g+1.
// A sub-block has only four possible values; they are rounded once each, parked in two registers
// as four halves, and every pair of weights is one byte-permute whose selector is the pair's two
// 2-bit codes times 0x22 plus 0x1010 (code c picks bytes 2c, 2c+1).
template <typename ab_t> struct Decoder<T_Q2_K, ab_t> {
  static constexpr int CORR_OFF = -1;
  static constexpr int RW = 10;   // 32 code bytes, the word holding the two scale bytes, (d, dmin): all 4-byte aligned
  static __device__ __forceinline__ void load(const uint8_t* row, int u, uint32_t (&raw)[RW]) {
    const uint32_t sb = smem_u32(row + (int64_t)(u >> 3) * 84);
    const int g = u & 7;
    const uint32_t sq = sb + 16 + 32 * (g >> 2);
#pragma unroll
    for (int i = 0; i < 8; ++i) raw[i] = lds32(sq + 4u * i);
    raw[8] = lds32(sb + ((2 * g) & ~3));
    raw[9] = lds32(sb + 80);
  }
  static __device__ __forceinline__ void decode(const uint8_t*, int u, const uint32_t (&raw)[RW], const DecodeCtx&, uint32_t (&out)[16]) {
    const int g = u & 7, sh = 2 * (g & 3);
    const float d = __half2float(__ushort_as_half((unsigned short)(raw[9] & 0xFFFFu)));
    const float dmin = __half2float(__ushort_as_half((unsigned short)(raw[9] >> 16)));
    const uint32_t sc2 = raw[8] >> (16 * (g & 1));
#pragma unroll
    for (int hb = 0; hb < 2; ++hb) {   // the two 16-value sub-blocks of the unit
      const uint32_t sc = (sc2 >> (8 * hb)) & 0xFFu;
      const float dl = d * (float)(sc & 0xFu), ml = dmin * (float)(sc >> 4);
      const uint32_t r0 = pack2<ab_t>(-ml, dl - ml), r1 = pack2<ab_t>(fmaf(2.f, dl, -ml), fmaf(3.f, dl, -ml));
#pragma unroll
      for (int i = 0; i < 4; ++i) {    // word 4hb + i: values 16hb + 4i .. + 3
        const uint32_t x = (raw[4 * hb + i] >> sh) & 0x03030303u;
        out[8 * hb + 2 * i] = __byte_perm(r0, r1, x * 0x22u + 0x1010u);
        out[8 * hb + 2 * i + 1] = __byte_perm(r0, r1, (x >> 16) * 0x22u + 0x1010u);
      }
    }
  }
  static __device__ __forceinline__ void corr(const uint8_t*, int, int64_t, uint32_t (&)[16]) {}
};

// ---- Q3_K: value = d * ((sc6 - 32) * (c - 4)), c = 2 low bits | hmask bit << 2; unit = 32-value group
// g = u&7 = 4n + j: bytes qs[32n..32n+31] >> 2j, bit g of hmask[0..31], scales 2g, 2g+1.  Blocks are
// 110 bytes, so everything is read as covering words and realigned.  The code lands at bits 3-5 of
// a byte (two rotates, two masks per four weights), one byte-permute per pair turns it into the
// half 128 + c (0x5800 | c << 3), one HFMA2 gives (c - 4) * sc exactly (|.| <= 128; the addend
// -132 * sc has 11 significant bits) and the multiplication by d rounds once.
template <typename ab_t> struct Decoder<T_Q3_K, ab_t> {
  static constexpr int CORR_OFF = -1;
  static constexpr int RW = 26;   // [0..9] code words, [10..19] hmask words, [20..24] the 12 scale bytes, [25] d
  static __device__ __forceinline__ void load(const uint8_t* row, int u, uint32_t (&raw)[RW]) {
    const uint8_t* blk = row + (int64_t)(u >> 3) * 110;
    const int g = u & 7;
    ldg_cover<9>(blk + 32 + 32 * (g >> 2), 32, raw);
    raw[9] = 0;
    ldg_cover<9>(blk, 32, raw + 10);
    raw[19] = 0;
    ldg_cover<4>(blk + 96, 12, raw + 20);
    raw[24] = 0;
    ldg_cover<1>(blk + 108, 2, raw + 25);
  }
  static __device__ __forceinline__ void decode(const uint8_t* row, int u, const uint32_t (&raw)[RW], const DecodeCtx&, uint32_t (&out)[16]) {
    static_assert(sizeof(ab_t) == 2 && std::is_same<ab_t, __half>::value, "Q3_K is decoded with fp16 arithmetic");
    const uint8_t* blk = row + (int64_t)(u >> 3) * 110;
    const int g = u & 7, k = g >> 1;
    const uint32_t sh_q = shift_of(blk + 32 + 32 * (g >> 2)), sh_h = shift_of(blk), sh_s = shift_of(blk + 96);
    // 6-bit scales 2g, 2g+1: low nibbles from byte 2g (mod 8) of the first eight scale bytes, shifted by
    // four for g >= 4; the two high bits from byte 2g mod 4 of the last four, bit pair g / 2
    const uint32_t a01 = word_at(raw + 20, k & 1, sh_s), tmp = word_at(raw + 20, 2, sh_s);
    const uint32_t us4 = ((a01 >> (4 * (k >> 1))) & 0x0F0F0F0Fu) | (((tmp >> (2 * k)) & 0x03030303u) << 4);
    const uint32_t us2 = us4 >> (16 * (g & 1));
    const uint32_t du = (raw[25] >> shift_of(blk + 108)) & 0xFFFFu;
    const __half2 d2 = u32_as_h2(du | (du << 16));
    const uint32_t rot_q = (uint32_t)(2 * (g & 3) - 3) & 31u, rot_h = (uint32_t)(g - 5) & 31u;
#pragma unroll
    for (int hb = 0; hb < 2; ++hb) {
      const __half s = __int2half_rn((int)((us2 >> (8 * hb)) & 0xFFu) - 32);
      const __half2 s2 = __half2half2(s), c2 = __half2half2(__hmul(s, __float2half_rn(-132.f)));
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t wq = word_at(raw, 4 * hb + i, sh_q), wh = word_at(raw + 10, 4 * hb + i, sh_h);
        const uint32_t c = (__funnelshift_r(wq, wq, rot_q) & 0x18181818u) | (__funnelshift_r(wh, wh, rot_h) & 0x20202020u);
        const __half2 p0 = u32_as_h2(__byte_perm(c, 0x58585858u, 0x4140)), p1 = u32_as_h2(__byte_perm(c, 0x58585858u, 0x4342));
        out[8 * hb + 2 * i] = h2_as_u32(hmul2_rn(__hfma2(p0, s2, c2), d2));
        out[8 * hb + 2 * i + 1] = h2_as_u32(hmul2_rn(__hfma2(p1, s2, c2), d2));
      }
    }
  }
  static __device__ __forceinline__ void corr(const uint8_t*, int, int64_t, uint32_t (&)[16]) {}
};

// ---- IQ4_XS: fp32 d*(ls-32)*level rounded once to ab_t; unit = 32-value group ib = u&7 -----------
template <typename ab_t> struct Decoder<T_IQ4_XS, ab_t> {
  static constexpr int CORR_OFF = -1;   // byte offset in a block of the fp16 that is the block's correction value (-1: none / computed)
  static constexpr int RW = 6;   // header (8 bytes) + 16 index bytes, 8-byte aligned
  static __device__ __forceinline__ void load(const uint8_t* row, int u, uint32_t (&raw)[RW]) {
    const uint8_t* blk = row + (int64_t)(u >> 3) * 136;
    const uint32_t sb = smem_u32(blk);
    const uint2 h = lds64(sb), a = lds64(sb + 8 + 16 * (u & 7)), b = lds64(sb + 16 + 16 * (u & 7));
    raw[0] = h.x; raw[1] = h.y; raw[2] = a.x; raw[3] = a.y; raw[4] = b.x; raw[5] = b.y;
  }
  static __device__ __forceinline__ void decode(const uint8_t*, int u, const uint32_t (&raw)[RW], const DecodeCtx& cx, uint32_t (&out)[16]) {
    const int ib = u & 7;
    const float d = __half2float(__ushort_as_half((unsigned short)(raw[0] & 0xffff)));
    const int ls = (int)(((raw[1] >> (4 * ib)) & 0xF) | ((((raw[0] >> 16) >> (2 * ib)) & 3) << 4)) - 32;
    const float dl = d * (float)ls;
#pragma unroll
    for (int i = 0; i < 4; ++i) {  // bytes 4i..4i+3: values 4i.. (low nibbles) and 16+4i.. (high)
      const uint32_t w = raw[2 + i];
      out[2 * i] = pack2<ab_t>(dl * cx.level(w & 0xF), dl * cx.level((w >> 8) & 0xF));
      out[2 * i + 1] = pack2<ab_t>(dl * cx.level((w >> 16) & 0xF), dl * cx.level((w >> 24) & 0xF));
      out[8 + 2 * i] = pack2<ab_t>(dl * cx.level((w >> 4) & 0xF), dl * cx.level((w >> 12) & 0xF));
      out[8 + 2 * i + 1] = pack2<ab_t>(dl * cx.level((w >> 20) & 0xF), dl * cx.level((w >> 28) & 0xF));
    }
  }
  static __device__ __forceinline__ void corr(const uint8_t*, int, int64_t, uint32_t (&)[16]) {}
};

// ---- IQ4_NL: fp32 d*level rounded once to ab_t; unit = one 18-byte block (2-byte aligned) ----------
template <typename ab_t> struct Decoder<T_IQ4_NL, ab_t> {
  static constexpr int CORR_OFF = -1;   // byte offset in a block of the fp16 that is the block's correction value (-1: none / computed)
  static constexpr int RW = 7;
  static __device__ __forceinline__ void load(const uint8_t* row, int u, uint32_t (&raw)[RW]) {
    ldg_cover<RW - 1>(row + (int64_t)u * 18, 18, raw);
    raw[RW - 1] = 0;
  }
  static __device__ __forceinline__ void decode(const uint8_t* row, int u, const uint32_t (&raw)[RW], const DecodeCtx& cx, uint32_t (&out)[16]) {
    const uint32_t sh = shift_of(row + (int64_t)u * 18);
    const float d = __half2float(__ushort_as_half((unsigned short)(word_at(raw, 0, sh) & 0xFFFFu)));
#pragma unroll
    for (int i = 0; i < 8; ++i) {  // stream half-word 1+i holds qs[2i], qs[2i+1]
      const int h = 1 + i;
      const uint32_t wv = word_at(raw, h >> 1, sh);
      const uint32_t t = (h & 1) ? (wv >> 16) : (wv & 0xFFFFu);
      out[i] = pack2<ab_t>(d * cx.level(t & 0xF), d * cx.level((t >> 8) & 0xF));
      out[8 + i] = pack2<ab_t>(d * cx.level((t >> 4) & 0xF), d * cx.level((t >> 12) & 0xF));
    }
  }
  static __device__ __forceinline__ void corr(const uint8_t*, int, int64_t, uint32_t (&)[16]) {}
};

// ---- IQ2_XXS: fp32 d*(0.5+s)*0.25*grid*sign rounded once; unit = 32-value group ib = u&7 ----------
// (value = +-round(d * magnitude): the product is formed in fp32 and rounded once, as in the
// reference; multiplying by -1.f afterwards is exact, so flipping the sign bit is the same)
template <typename ab_t> struct Decoder<T_IQ2_XXS, ab_t> {
  static constexpr int CORR_OFF = -1;   // byte offset in a block of the fp16 that is the block's correction value (-1: none / computed)
  static constexpr int RW = 5;   // [0] word holding d, [1..3] the group's 8 bytes (+ cover), [4] pad
  static __device__ __forceinline__ void load(const uint8_t* row, int u, uint32_t (&raw)[RW]) {
    const uint8_t* blk = row + (int64_t)(u >> 3) * 66;
    ldg_cover<1>(blk, 2, raw);
    ldg_cover<3>(blk + 2 + 8 * (u & 7), 8, raw + 1);
    raw[4] = 0;
  }
  static __device__ __forceinline__ void decode(const uint8_t* row, int u, const uint32_t (&raw)[RW], const DecodeCtx& cx, uint32_t (&out)[16]) {
    const uint8_t* blk = row + (int64_t)(u >> 3) * 66;
    const float dh = __half2float(__ushort_as_half((unsigned short)((raw[0] >> shift_of(blk)) & 0xFFFFu)));
    const uint32_t sh = shift_of(blk + 2 + 8 * (u & 7));
    const uint32_t idx = word_at(raw + 1, 0, sh), aux = word_at(raw + 1, 1, sh);
    const float d = dh * (0.5f + (float)(aux >> 28)) * 0.25f;
    // the three possible magnitudes of this group, each rounded once (the sign flips only the top bit)
    const uint32_t r0 = pack2<ab_t>(d * 8.f, d * 25.f), r1 = pack2<ab_t>(d * 43.f, 0.f);
#pragma unroll
    for (int il = 0; il < 4; ++il) {
      const uint2 sel = cx.sel_at((idx >> (8 * il)) & 0xFF);
      const uint4 sg = cx.sgn_at((aux >> (7 * il)) & 127);
      out[4 * il + 0] = __byte_perm(r0, r1, sel.x) ^ sg.x;
      out[4 * il + 1] = __byte_perm(r0, r1, sel.x >> 16) ^ sg.y;
      out[4 * il + 2] = __byte_perm(r0, r1, sel.y) ^ sg.z;
      out[4 * il + 3] = __byte_perm(r0, r1, sel.y >> 16) ^ sg.w;
    }
  }
  static __device__ __forceinline__ void corr(const uint8_t*, int, int64_t, uint32_t (&)[16]) {}
};

// =============================================================================================
// Whole-stage decoders: one thread turns the 64 values of one weight row of one K stage into
// the 128 bytes of that row in the A tile (out[4c..4c+3] = 16-byte piece c of the row).
//
// The specialised ("fast") forms read a dense 256-value chunk of the row from shared memory
// (the 2-D TMA box of mmq.cu) with 16-byte loads at compile-time offsets and build fp16 pairs
// with the mantissa trick: OR-ing a small unsigned integer n into the mantissa of 1024.0
// (0x6400) gives exactly 1024 + n, into bits 4-7 of 64.0 (0x5400) exactly 64 + n.  Values are
// the same as the 32-value decoders above produce (one rounding, in the final multiply).
//
// PERM: order of the 64 values inside the stage.  0 = natural.  1 = within every group of four
// consecutive values the middle two are swapped (0,2,1,3): the two low nibbles that sit 16 bits
// apart in a 32-bit word of packed bytes become one fp16 pair with a single AND/OR.  The
// activation matrix is written in the same order (quantize_q8_1.cu), so the contraction is
// unchanged.
// =============================================================================================
template <int TYPE, typename ab_t> struct Stage64 {
  static constexpr bool FAST = false;
  static constexpr int PERM = 0;
};

__device__ __forceinline__ uint4 lds128(const uint8_t* p) { return lds128s(smem_u32(p)); }
__device__ __forceinline__ __half2 h2const(float v) { return __floats2half2_rn(v, v); }

// ---- Q4_K: chunk = one 144-byte super-block; stage SC = sub-blocks 2SC (low nibbles) and 2SC+1 ----
template <> struct Stage64<T_Q4_K, __half> {
  static constexpr bool FAST = true;
  static constexpr int PERM = 1;
  template <int SC> static __device__ __forceinline__ void decode(const uint8_t* blk, uint32_t (&out)[32]) {
    const uint4 h = lds128(blk);
    const uint4 qa = lds128(blk + 16 + 32 * SC), qb = lds128(blk + 32 + 32 * SC);
    const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
    const __half dall = __ushort_as_half((unsigned short)(h.x & 0xffff));
    int sc0, sc1, m;
    q4k_scale_min(h.y, h.z, h.w, 2 * SC, sc0, m);
    q4k_scale_min(h.y, h.z, h.w, 2 * SC + 1, sc1, m);
    const __half d0 = __hmul_rn(dall, __int2half_rn(sc0)), d1 = __hmul_rn(dall, __int2half_rn(sc1));
    const __half2 s0 = __half2half2(d0), s1 = __half2half2(d1);
    const float big = fmaxf(fabsf(__half2float(d0)), fabsf(__half2float(d1)));
    if (big < 32.f) {
      // (1024 + n) * s - 1024 * s: the product term is exact, so this is n * s rounded once
      const __half2 c0 = __hmul2_rn(s0, h2const(-1024.f)), c1 = __hmul2_rn(s1, h2const(-64.f));
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t a = w[j], b = w[j] >> 8;
        out[2 * j] = h2_as_u32(__hfma2(u32_as_h2((a & 0x000F000Fu) | 0x64006400u), s0, c0));
        out[2 * j + 1] = h2_as_u32(__hfma2(u32_as_h2((b & 0x000F000Fu) | 0x64006400u), s0, c0));
        out[16 + 2 * j] = h2_as_u32(__hfma2(u32_as_h2((a & 0x00F000F0u) | 0x54005400u), s1, c1));
        out[16 + 2 * j + 1] = h2_as_u32(__hfma2(u32_as_h2((b & 0x00F000F0u) | 0x54005400u), s1, c1));
      }
    } else {  // 1024 * s would overflow fp16: subtract the offset first (exact), then scale
      const __half2 o0 = h2const(1024.f), o1 = h2const(64.f);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t a = w[j], b = w[j] >> 8;
        out[2 * j] = h2_as_u32(hmul2_rn(__hsub2(u32_as_h2((a & 0x000F000Fu) | 0x64006400u), o0), s0));
        out[2 * j + 1] = h2_as_u32(hmul2_rn(__hsub2(u32_as_h2((b & 0x000F000Fu) | 0x64006400u), o0), s0));
        out[16 + 2 * j] = h2_as_u32(hmul2_rn(__hsub2(u32_as_h2((a & 0x00F000F0u) | 0x54005400u), o1), s1));
        out[16 + 2 * j + 1] = h2_as_u32(hmul2_rn(__hsub2(u32_as_h2((b & 0x00F000F0u) | 0x54005400u), o1), s1));
      }
    }
  }
};

// ---- Q5_K: chunk = one 176-byte super-block (d, dmin, 12 scale bytes, 32 bytes of fifth bits, 128 bytes of
// nibbles); stage SC = sub-blocks 2SC (low nibbles of qs[32SC..], bit 2SC of qh[l]) and 2SC+1 (high nibbles,
// bit 2SC+1).  As Q4_K with one more AND/OR per pair: the fifth bit lands at mantissa bit 4 of 1024 + n
// (low nibbles) or at mantissa bit 8 of 64 + n / 16 (high nibbles, n sits four bits up).
template <> struct Stage64<T_Q5_K, __half> {
  static constexpr bool FAST = true;
  static constexpr int PERM = 1;
  template <int SC> static __device__ __forceinline__ void decode(const uint8_t* blk, uint32_t (&out)[32]) {
    const uint4 h = lds128(blk);
    const uint4 ha = lds128(blk + 16), hb = lds128(blk + 32);
    const uint4 qa = lds128(blk + 48 + 32 * SC), qb = lds128(blk + 64 + 32 * SC);
    const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
    const uint32_t hw[8] = {ha.x, ha.y, ha.z, ha.w, hb.x, hb.y, hb.z, hb.w};
    const __half dall = __ushort_as_half((unsigned short)(h.x & 0xffff));
    int sc0, sc1, m;
    q4k_scale_min(h.y, h.z, h.w, 2 * SC, sc0, m);
    q4k_scale_min(h.y, h.z, h.w, 2 * SC + 1, sc1, m);
    const __half d0 = __hmul_rn(dall, __int2half_rn(sc0)), d1 = __hmul_rn(dall, __int2half_rn(sc1));
    const __half2 s0 = __half2half2(d0), s1 = __half2half2(d1);
    const float big = fmaxf(fabsf(__half2float(d0)), fabsf(__half2float(d1)));
    if (big < 32.f) {
      // (1024 + n) * s - 1024 * s: the product term is exact, so this is n * s rounded once
      const __half2 c0 = __hmul2_rn(s0, h2const(-1024.f)), c1 = __hmul2_rn(s1, h2const(-64.f));
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t a = w[j], b = w[j] >> 8;
        const uint32_t x = hw[j] >> (2 * SC), y = hw[j] >> (2 * SC + 8);   // fifth bits of values (4j, 4j+2) / (4j+1, 4j+3) at bits 0 and 16
        out[2 * j] = h2_as_u32(__hfma2(u32_as_h2((a & 0x000F000Fu) | ((x << 4) & 0x00100010u) | 0x64006400u), s0, c0));
        out[2 * j + 1] = h2_as_u32(__hfma2(u32_as_h2((b & 0x000F000Fu) | ((y << 4) & 0x00100010u) | 0x64006400u), s0, c0));
        out[16 + 2 * j] = h2_as_u32(__hfma2(u32_as_h2((a & 0x00F000F0u) | ((x << 7) & 0x01000100u) | 0x54005400u), s1, c1));
        out[16 + 2 * j + 1] = h2_as_u32(__hfma2(u32_as_h2((b & 0x00F000F0u) | ((y << 7) & 0x01000100u) | 0x54005400u), s1, c1));
      }
    } else {  // 1024 * s would overflow fp16: subtract the offset first (exact), then scale
      const __half2 o0 = h2const(1024.f), o1 = h2const(64.f);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t a = w[j], b = w[j] >> 8;
        const uint32_t x = hw[j] >> (2 * SC), y = hw[j] >> (2 * SC + 8);
        out[2 * j] = h2_as_u32(hmul2_rn(__hsub2(u32_as_h2((a & 0x000F000Fu) | ((x << 4) & 0x00100010u) | 0x64006400u), o0), s0));
        out[2 * j + 1] = h2_as_u32(hmul2_rn(__hsub2(u32_as_h2((b & 0x000F000Fu) | ((y << 4) & 0x00100010u) | 0x64006400u), o0), s0));
        out[16 + 2 * j] = h2_as_u32(hmul2_rn(__hsub2(u32_as_h2((a & 0x00F000F0u) | ((x << 7) & 0x01000100u) | 0x54005400u), o1), s1));
        out[16 + 2 * j + 1] = h2_as_u32(hmul2_rn(__hsub2(u32_as_h2((b & 0x00F000F0u) | ((y << 7) & 0x01000100u) | 0x54005400u), o1), s1));
      }
    }
  }
};

// ---- Q4_0: chunk = 8 blocks of 18 bytes; stage SC = blocks 2SC, 2SC+1 at byte 36*SC ----------------
template <> struct Stage64<T_Q4_0, __half> {
  static constexpr bool FAST = true;
  static constexpr int PERM = 1;
  // The operand is half(q * d) with the UNSIGNED code q = 0..15 (the "- 8" of the format rides in the
  // correction column: -8 * d * s8, which is the reference's own tiled formula d * (sumi * d8 - 8 * s8),
  // vecdotq.cuh:61-64), so one HFMA2 makes a pair: (1024 + q) * d - 1024 * d is q * d rounded once.
  static __device__ __forceinline__ void block(const uint32_t (&q)[4], __half2 d2, uint32_t* out) {
    const float ad = fabsf(__low2float(d2));
    if (ad < 32.f) {
      const __half2 c0 = __hmul2_rn(d2, h2const(-1024.f)), c1 = __hmul2_rn(d2, h2const(-64.f));   // exact
#pragma unroll
      for (int j = 0; j < 4; ++j) {   // bytes 4j..4j+3: low nibbles = values 4j.., high nibbles = values 16+4j..
        const uint32_t a = q[j], b = q[j] >> 8;
        out[2 * j] = h2_as_u32(__hfma2(u32_as_h2((a & 0x000F000Fu) | 0x64006400u), d2, c0));
        out[2 * j + 1] = h2_as_u32(__hfma2(u32_as_h2((b & 0x000F000Fu) | 0x64006400u), d2, c0));
        out[8 + 2 * j] = h2_as_u32(__hfma2(u32_as_h2((a & 0x00F000F0u) | 0x54005400u), d2, c1));
        out[8 + 2 * j + 1] = h2_as_u32(__hfma2(u32_as_h2((b & 0x00F000F0u) | 0x54005400u), d2, c1));
      }
    } else {   // 1024 * d would overflow fp16: subtract the offset first (exact), then scale
      const __half2 o0 = h2const(1024.f), o1 = h2const(64.f);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t a = q[j], b = q[j] >> 8;
        out[2 * j] = h2_as_u32(hmul2_rn(__hsub2(u32_as_h2((a & 0x000F000Fu) | 0x64006400u), o0), d2));
        out[2 * j + 1] = h2_as_u32(hmul2_rn(__hsub2(u32_as_h2((b & 0x000F000Fu) | 0x64006400u), o0), d2));
        out[8 + 2 * j] = h2_as_u32(hmul2_rn(__hsub2(u32_as_h2((a & 0x00F000F0u) | 0x54005400u), o1), d2));
        out[8 + 2 * j + 1] = h2_as_u32(hmul2_rn(__hsub2(u32_as_h2((b & 0x00F000F0u) | 0x54005400u), o1), d2));
      }
    }
  }
  template <int SC> static __device__ __forceinline__ void decode(const uint8_t* chunk, uint32_t (&out)[32]) {
    constexpr int A0 = (36 * SC) & ~15, O = (36 * SC - A0) / 4;   // aligned start, word offset of block 2SC
    uint32_t W[12];
#pragma unroll
    for (int i = 0; i < 3; ++i) {
      const uint4 v = lds128(chunk + A0 + 16 * i);
      W[4 * i] = v.x; W[4 * i + 1] = v.y; W[4 * i + 2] = v.z; W[4 * i + 3] = v.w;
    }
    // block 2SC starts at word O (d in the low half, nibbles 2 bytes in); block 2SC+1 at word O+4, upper half
    const uint32_t da = W[O] & 0xFFFFu, db = W[O + 4] >> 16;
    const uint32_t qa[4] = {__funnelshift_r(W[O], W[O + 1], 16), __funnelshift_r(W[O + 1], W[O + 2], 16),
                            __funnelshift_r(W[O + 2], W[O + 3], 16), __funnelshift_r(W[O + 3], W[O + 4], 16)};
    const uint32_t qb[4] = {W[O + 5], W[O + 6], W[O + 7], W[O + 8]};
    block(qa, u32_as_h2(da | (da << 16)), out);
    block(qb, u32_as_h2(db | (db << 16)), out + 16);
  }
};

// ---- Q8_0: chunk = 8 blocks of 34 bytes; stage SC = blocks 2SC, 2SC+1 at byte 68*SC ----------------
template <> struct Stage64<T_Q8_0, __half> {
  static constexpr bool FAST = true;
  static constexpr int PERM = 0;
  // two int8 codes (already biased by +128) -> (1024 + u0, 1024 + u1) -> (u - 128) * d
  static __device__ __forceinline__ uint32_t pair(uint32_t w, uint32_t sel, __half2 d2) {
    const __half2 o = h2const(1152.f);
    return h2_as_u32(hmul2_rn(__hsub2(u32_as_h2(__byte_perm(w, 0x64646464u, sel)), o), d2));
  }
  template <int SC> static __device__ __forceinline__ void decode(const uint8_t* chunk, uint32_t (&out)[32]) {
    constexpr int A0 = (68 * SC) & ~15, O = (68 * SC - A0) / 4;
    uint32_t W[20];
#pragma unroll
    for (int i = 0; i < 5; ++i) {
      const uint4 v = lds128(chunk + A0 + 16 * i);
      W[4 * i] = v.x; W[4 * i + 1] = v.y; W[4 * i + 2] = v.z; W[4 * i + 3] = v.w;
    }
    const uint32_t da = W[O] & 0xFFFFu, db = W[O + 8] >> 16;
    const __half2 d2a = u32_as_h2(da | (da << 16)), d2b = u32_as_h2(db | (db << 16));
    // block 2SC: codes start in the upper half of word O; pair t = codes 2t, 2t+1 = half-word 1+t of the block
#pragma unroll
    for (int t = 0; t < 16; ++t) {
      const uint32_t wv = W[O + ((1 + t) >> 1)] ^ 0x80808080u;
      out[t] = pair(wv, ((1 + t) & 1) ? 0x4342u : 0x4140u, d2a);
    }
    // block 2SC+1: codes start at word O+9, aligned
#pragma unroll
    for (int t = 0; t < 16; ++t) {
      const uint32_t wv = W[O + 9 + (t >> 1)] ^ 0x80808080u;
      out[16 + t] = pair(wv, (t & 1) ? 0x4342u : 0x4140u, d2b);
    }
  }
};

}  // namespace gguf_b200
