// Decode GEMV for one or two activation vectors, the latency-critical case:
// Y[m][n] = sum_k dequant(W)[n,k] * q8_1(x_m)[k].  Also serves MoE decode (one grid row per
// (token, expert) pair) and the tensor-parallel form that forwards its slice to peer GPUs.
// Same arithmetic as gemv.cu (reference: mul_mat_vec_q, mmvq.cuh:2-41 and vec_dot_*_q8_1 of
// vecdotq.cuh), specialised so that the inner loop spends its instructions on the weights only:
//
//  * Lane l of a warp always works on the same K positions (units l, l+32, ... of the warp's
//    K-slice) for every row, so the activations it needs -- int8 codes and {d, sum} -- are loaded
//    ONCE into registers at kernel start and never touched in shared memory again.
//  * Long rows are split into KS in {1,2,4,8} K-slices handled by different warps of the CTA so
//    that a lane's activation slice always fits in registers; the per-slice partial sums meet in
//    shared memory and are added in a fixed order (deterministic) every 32 row iterations.
//  * Weights stream exactly as in gemv.cu: one 1-D bulk copy (TMA) per (row, slice) into a
//    per-warp ring of stages, mbarrier completion, 16-byte rounded starts for the 2-byte aligned
//    formats, bounded waits.
//  * The unit loop is unrolled at compile time and integer dots run on independent dp4a chains.
#include <type_traits>

#include "common.cuh"
#include "kernels.h"
#include "q8_1_lane.cuh"
#include "tables.cuh"

namespace gguf_b200 {

constexpr int G1_WARPS = 8;
constexpr int G1_BATCH = 32;   // row iterations between two flushes of the slice partials
constexpr int G1_TAB_COPIES = 16;   // bank-conflict-free copies of the IQ2_XXS code books (see the kernel)

__device__ __forceinline__ __half2 u32_as_half2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }
__device__ __forceinline__ int dp4a_us1(uint32_t a, uint32_t b, int c) {
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
// `blk` below is the 32-bit shared-window address of a weight block (all loads stay in that window).
// The loads of the decoders are asm statements WITHOUT `volatile`: to the compiler they are pure
// functions of the address, so the two dot products of a two-vector kernel share one set of loads
// and one header decode, and loads of different units may be moved next to each other.  What keeps
// them behind the arrival of the data is a data dependency: every address derives from
// fresh_stage(), a volatile statement placed after the barrier wait.
__device__ __forceinline__ uint32_t fresh_stage(uint32_t a) {
  uint32_t r;
  asm volatile("mov.u32 %0, %1;" : "=r"(r) : "r"(a) : "memory");
  return r;
}
__device__ __forceinline__ uint32_t pl32(uint32_t a) {
  uint32_t v;
  asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint2 pl64(uint32_t a) {
  uint2 v;
  asm("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
  return v;
}
__device__ __forceinline__ uint4 pl128(uint32_t a) {
  uint4 v;
  asm("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t pl16(uint32_t a) {
  unsigned short h;
  asm("ld.shared.u16 %0, [%1];" : "=h"(h) : "r"(a));
  return h;
}
__device__ __forceinline__ float plh(uint32_t a) { return __half2float(__ushort_as_half((unsigned short)pl16(a))); }
// N consecutive words from an address that is only 2-byte aligned: the N + 1 aligned words that
// cover them, realigned with funnel shifts
template <int N> __device__ __forceinline__ void lds_a2(uint32_t a, uint32_t (&w)[N]) {
  const uint32_t al = a & ~3u, sh = (a & 3u) * 8u;
  uint32_t r[N + 1];
#pragma unroll
  for (int i = 0; i <= N; ++i) r[i] = pl32(al + 4u * i);
#pragma unroll
  for (int i = 0; i < N; ++i) w[i] = __funnelshift_r(r[i], r[i + 1], sh);
}

struct Tab1 {
  uint32_t grid;    // shared-window addresses of this lane's copies of the IQ2_XXS code books
  uint32_t smask;
  uint32_t kv[4];
};

// Per type: UPB units per block, XW activation words and XD floats held per unit.
template <int TYPE> struct G1;

// ---- Q8_0: unit = block of 32 -----------------------------------------------------------
template <> struct G1<T_Q8_0> {
  static constexpr int UPB = 1, XW = 8, XD = 2, UMAX = 4;
  static __device__ __forceinline__ void load_x(const uint8_t* qs, const float2* ds, int u, int, uint32_t (&x)[XW], float (&xd)[XD]) {
    const uint4* p = reinterpret_cast<const uint4*>(qs + (size_t)u * 32);
    const uint4 a = p[0], b = p[1];   // plain loads: the quantized activations may be in shared memory
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
    const float2 d = ds[u];
    xd[0] = d.x; xd[1] = d.y;
  }
  static __device__ __forceinline__ float unit(uint32_t blk, int, const uint32_t (&x)[XW], const float (&xd)[XD], const Tab1&) {
    const float d = plh(blk);
    uint32_t w[8];
    lds_a2<8>(blk + 2, w);
    int s0 = 0, s1 = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      s0 = __dp4a((int)w[2 * i], (int)x[2 * i], s0);
      s1 = __dp4a((int)w[2 * i + 1], (int)x[2 * i + 1], s1);
    }
    return d * xd[0] * (float)(s0 + s1);
  }
};

// ---- Q4_0 -------------------------------------------------------------------------------
template <> struct G1<T_Q4_0> {
  static constexpr int UPB = 1, XW = 8, XD = 2, UMAX = 4;
  static __device__ __forceinline__ void load_x(const uint8_t* qs, const float2* ds, int u, int b, uint32_t (&x)[XW], float (&xd)[XD]) {
    G1<T_Q8_0>::load_x(qs, ds, u, b, x, xd);
  }
  static __device__ __forceinline__ float unit(uint32_t blk, int, const uint32_t (&x)[XW], const float (&xd)[XD], const Tab1&) {
    const float d = plh(blk);
    uint32_t q[4];
    lds_a2<4>(blk + 2, q);
    int lo = 0, hi = 0;  // hi = 16 * (high-nibble dot): nibbles stay in place
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      lo = dp4a_us1(q[i] & 0x0F0F0F0Fu, x[i], lo);
      hi = dp4a_us1(q[i] & 0xF0F0F0F0u, x[4 + i], hi);
    }
    return d * ((float)(lo + (hi >> 4)) * xd[0] - 8.0f * xd[1]);
  }
};

// ---- Q4_K: unit p = 64 values (sub-blocks 2p, 2p+1) --------------------------------------
template <> struct G1<T_Q4_K> {
  static constexpr int UPB = 4, XW = 16, XD = 4, UMAX = 2;
  static __device__ __forceinline__ void load_x(const uint8_t* qs, const float2* ds, int u, int, uint32_t (&x)[XW], float (&xd)[XD]) {
    const uint4* p = reinterpret_cast<const uint4*>(qs + (size_t)u * 64);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 a = p[i];
      x[4 * i] = a.x; x[4 * i + 1] = a.y; x[4 * i + 2] = a.z; x[4 * i + 3] = a.w;
    }
    const float4 d = *reinterpret_cast<const float4*>(ds + 2 * u);
    xd[0] = d.x; xd[1] = d.y; xd[2] = d.z; xd[3] = d.w;  // d8_0, d8_0*sum0, d8_1, d8_1*sum1
  }
  static __device__ __forceinline__ float unit(uint32_t blk, int p, const uint32_t (&x)[XW], const float (&xd)[XD], const Tab1&) {
    const uint4 hdr = pl128(blk);
    const __half2 dm = *reinterpret_cast<const __half2*>(&hdr.x);
    const float d = __low2float(dm), dmin = __high2float(dm);
    const int sh = 16 * (p & 1);
    const uint32_t a = hdr.y >> sh, b = hdr.z >> sh, c = hdr.w >> sh;
    // get_scale_min_k4: both cases computed and merged with a mask (lanes of a warp differ in p:
    // a branch here would run both sides one after the other)
    const uint32_t lowm = p < 2 ? 0xFFFFFFFFu : 0u;
    const uint32_t sc2 = ((a & 0x3F3Fu) & lowm) | (((c & 0x0F0Fu) | ((a >> 2) & 0x3030u)) & ~lowm);
    const uint32_t mn2 = ((b & 0x3F3Fu) & lowm) | ((((c >> 4) & 0x0F0Fu) | ((b >> 2) & 0x3030u)) & ~lowm);
    const int sc0 = sc2 & 0xFF, sc1 = (sc2 >> 8) & 0xFF;
    const float m0 = (float)(mn2 & 0xFF), m1 = (float)((mn2 >> 8) & 0xFF);
    const uint4 qa = pl128(blk + 16 + 32 * p), qb = pl128(blk + 32 + 32 * p);
    const uint32_t q[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
    int a0 = 0, a1 = 0, b0 = 0, b1 = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      a0 = dp4a_us1(q[2 * i] & 0x0F0F0F0Fu, x[2 * i], a0);
      a1 = dp4a_us1(q[2 * i + 1] & 0x0F0F0F0Fu, x[2 * i + 1], a1);
      b0 = dp4a_us1(q[2 * i] & 0xF0F0F0F0u, x[8 + 2 * i], b0);
      b1 = dp4a_us1(q[2 * i + 1] & 0xF0F0F0F0u, x[8 + 2 * i + 1], b1);
    }
    return d * (xd[0] * (float)((a0 + a1) * sc0) + xd[2] * (float)(((b0 + b1) >> 4) * sc1)) - dmin * (xd[1] * m0 + xd[3] * m1);
  }
};

// ---- Q6_K: unit u4: half ip = u4>>1, column half h = u4&1 -> groups 4ip+h and 4ip+2+h -------
// The codes stay unsigned (0..63); the "-32" is applied through the activation sums of each
// 16-value sub-block, which are constants of the lane (xs packs them: 4 x int16 in XW words 16,17).
template <> struct G1<T_Q6_K> {
  static constexpr int UPB = 4, XW = 18, XD = 2, UMAX = 2;
  static __device__ __forceinline__ void load_x(const uint8_t* qs, const float2* ds, int u, int, uint32_t (&x)[XW], float (&xd)[XD]) {
    const int b = u >> 2, u4 = u & 3, ip = u4 >> 1, h = u4 & 1;
    const int ga = 8 * b + 4 * ip + h, gb = ga + 2;
    const uint4* pa = reinterpret_cast<const uint4*>(qs + (size_t)ga * 32);
    const uint4* pb = reinterpret_cast<const uint4*>(qs + (size_t)gb * 32);
    const uint4 a0 = pa[0], a1 = pa[1], b0 = pb[0], b1 = pb[1];
    x[0] = a0.x; x[1] = a0.y; x[2] = a0.z; x[3] = a0.w; x[4] = a1.x; x[5] = a1.y; x[6] = a1.z; x[7] = a1.w;
    x[8] = b0.x; x[9] = b0.y; x[10] = b0.z; x[11] = b0.w; x[12] = b1.x; x[13] = b1.y; x[14] = b1.z; x[15] = b1.w;
    int s[4] = {0, 0, 0, 0};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      s[0] = __dp4a(0x01010101, (int)x[i], s[0]);
      s[1] = __dp4a(0x01010101, (int)x[4 + i], s[1]);
      s[2] = __dp4a(0x01010101, (int)x[8 + i], s[2]);
      s[3] = __dp4a(0x01010101, (int)x[12 + i], s[3]);
    }
    x[16] = ((uint32_t)s[0] & 0xFFFFu) | ((uint32_t)s[1] << 16);
    x[17] = ((uint32_t)s[2] & 0xFFFFu) | ((uint32_t)s[3] << 16);
    xd[0] = ds[ga].x;
    xd[1] = ds[gb].x;
  }
  static __device__ __forceinline__ float unit(uint32_t blk, int u4, const uint32_t (&x)[XW], const float (&xd)[XD], const Tab1&) {
    const int ip = u4 >> 1, h = u4 & 1;
    uint32_t ql[8], qh[8];
    lds_a2<8>(blk + 64 * ip + 32 * h, ql);
    lds_a2<8>(blk + 128 + 32 * ip, qh);
    // the scale pairs sit at even offsets of a 2-byte aligned block: two 16-bit loads
    const uint32_t sca = pl16(blk + 192 + 8 * ip + 2 * h), scb = pl16(blk + 196 + 8 * ip + 2 * h);
    const int sa0 = (int)(int8_t)(sca & 0xFF), sa1 = (int)(int8_t)(sca >> 8), sb0 = (int)(int8_t)(scb & 0xFF), sb1 = (int)(int8_t)(scb >> 8);
    const float d = plh(blk + 208);
    const int s2 = 2 * h;
    int a0 = 0, a1 = 0, b0 = 0, b1 = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t hh = qh[i] >> s2;  // bits 0-1 of each byte: group A, bits 4-5: group B
      const uint32_t va = (ql[i] & 0x0F0F0F0Fu) | ((hh << 4) & 0x30303030u);
      const uint32_t vb = ((ql[i] >> 4) & 0x0F0F0F0Fu) | (hh & 0x30303030u);
      if (i < 4) {
        a0 = dp4a_us1(va, x[i], a0);
        b0 = dp4a_us1(vb, x[8 + i], b0);
      } else {
        a1 = dp4a_us1(va, x[i], a1);
        b1 = dp4a_us1(vb, x[8 + i], b1);
      }
    }
    const int xs0 = (int)(short)(x[16] & 0xFFFF), xs1 = (int)(short)(x[16] >> 16);
    const int xs2 = (int)(short)(x[17] & 0xFFFF), xs3 = (int)(short)(x[17] >> 16);
    const int ia = (a0 - 32 * xs0) * sa0 + (a1 - 32 * xs1) * sa1;
    const int ib = (b0 - 32 * xs2) * sb0 + (b1 - 32 * xs3) * sb1;
    return d * (xd[0] * (float)ia + xd[1] * (float)ib);
  }
};

// ---- IQ4_XS: unit ib = 32 values -------------------------------------------------------------
// The 16 levels live in four registers.  One byte-permute picks four bytes out of eight by four
// 3-bit selectors, so a 4-bit index takes two permutes (levels 0-7, levels 8-15) and a third that
// chooses between them by bit 3 -- and the packed weight word itself serves as the selector: its
// nibbles are (value b, value 16+b) for each byte b.  The level bytes therefore come out in the
// order (v, v+16, v+1, v+17); instead of sorting them back, the lane's activations are shuffled
// into that order once, when they are loaded.
template <> struct G1<T_IQ4_XS> {
  static constexpr int UPB = 8, XW = 8, XD = 2, UMAX = 4;
  static __device__ __forceinline__ void load_x(const uint8_t* qs, const float2* ds, int u, int b, uint32_t (&x)[XW], float (&xd)[XD]) {
    uint32_t n[8];
    G1<T_Q8_0>::load_x(qs, ds, u, b, n, xd);
#pragma unroll
    for (int i = 0; i < 4; ++i) {   // n[i] = values 4i..4i+3, n[4+i] = values 16+4i..
      x[2 * i] = __byte_perm(n[i], n[4 + i], 0x5140);       // (4i, 16+4i, 4i+1, 16+4i+1)
      x[2 * i + 1] = __byte_perm(n[i], n[4 + i], 0x7362);   // (4i+2, 16+4i+2, 4i+3, 16+4i+3)
    }
  }
  // levels of the four 4-bit indices in the low 16 bits of q3 (bit 3 of each cleared) / sel (which half)
  static __device__ __forceinline__ uint32_t lut4(uint32_t q3, uint32_t sel, const Tab1& t) {
    return __byte_perm(__byte_perm(t.kv[0], t.kv[1], q3), __byte_perm(t.kv[2], t.kv[3], q3), sel);
  }
  static __device__ __forceinline__ float unit(uint32_t blk, int ib, const uint32_t (&x)[XW], const float (&xd)[XD], const Tab1& t) {
    const uint2 hdr = pl64(blk);
    const float d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xffff)));
    const int ls = (int)(((hdr.y >> (4 * ib)) & 0xF) | ((((hdr.x >> 16) >> (2 * ib)) & 3) << 4)) - 32;
    const uint2 qa = pl64(blk + 8 + 16 * ib), qb = pl64(blk + 16 + 16 * ib);
    const uint32_t q[4] = {qa.x, qa.y, qb.x, qb.y};
    int s0 = 0, s1 = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t q3 = q[i] & 0x77777777u;                                  // selectors within a half of the table
      const uint32_t sel = ((q[i] & 0x88888888u) >> 1) | 0x32103210u;          // nibble j: j (low half) or j + 4 (high half)
      s0 = __dp4a((int)lut4(q3, sel, t), (int)x[2 * i], s0);
      s1 = __dp4a((int)lut4(q3 >> 16, sel >> 16, t), (int)x[2 * i + 1], s1);
    }
    return d * (float)ls * xd[0] * (float)(s0 + s1);
  }
};

// ---- IQ2_XXS: unit ib = 32 values ------------------------------------------------------------
template <> struct G1<T_IQ2_XXS> {
  static constexpr int UPB = 8, XW = 8, XD = 2, UMAX = 4;
  static __device__ __forceinline__ void load_x(const uint8_t* qs, const float2* ds, int u, int b, uint32_t (&x)[XW], float (&xd)[XD]) {
    G1<T_Q8_0>::load_x(qs, ds, u, b, x, xd);
  }
  static __device__ __forceinline__ float unit(uint32_t blk, int ib, const uint32_t (&x)[XW], const float (&xd)[XD], const Tab1& t) {
    const float d = plh(blk);
    uint32_t q[2];
    lds_a2<2>(blk + 2 + 8 * ib, q);
    const uint32_t aux = q[1];
    int sp = 0, sn = 0;
#pragma unroll
    for (int il = 0; il < 4; ++il) {
      const uint2 gr = pl64(t.grid + ((q[0] >> (8 * il)) & 0xFF) * (8 * G1_TAB_COPIES));     // this lane's copy of the entry
      const uint2 sm = pl64(t.smask + ((aux >> (7 * il)) & 127) * (8 * G1_TAB_COPIES));
      sp = dp4a_us1(gr.x, x[2 * il], sp);
      sp = dp4a_us1(gr.y, x[2 * il + 1], sp);
      sn = dp4a_us1(gr.x & sm.x, x[2 * il], sn);
      sn = dp4a_us1(gr.y & sm.y, x[2 * il + 1], sn);
    }
    return d * (0.5f + (float)(aux >> 28)) * 0.25f * xd[0] * (float)(sp - 2 * sn);
  }
};

// ---- the other code-book types: IQ2_XS, IQ2_S, IQ3_XXS, IQ3_S, IQ1_S, IQ1_M ---------------------
// unit ib = 32 values (one q8_1 block).  Their code books (1 to 8 KB each) are read from global
// memory through the read-only path, as the reference's vec_dot_iq*_q8_1 do (vecdotq.cuh:1554-1750):
// these formats trade arithmetic for size and are bound by the look-ups, not by the weight stream.
__device__ __forceinline__ uint32_t pl8(uint32_t a) {
  uint32_t v;
  asm("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
// bit j of a nibble -> byte j of a word all ones (the reference's __vcmpeq4 form, vecdotq.cuh:1598-1599)
__device__ __forceinline__ uint32_t sign_mask4(uint32_t nib) { return __vcmpeq4(((nib & 0xfu) * 0x01010101u) & 0x08040201u, 0x08040201u); }
// seven sign bits + the eighth that makes the parity even (the ksigns_iq2xs table, computed)
__device__ __forceinline__ uint32_t signs_from7(uint32_t s7) { return s7 | ((__popc(s7) & 1u) << 7); }
// dot product of eight signed code-book magnitudes (two words, sign bit j = value j negative) with eight int8 activations
__device__ __forceinline__ int dot8_signed(uint32_t g0, uint32_t g1, uint32_t signs, uint32_t x0, uint32_t x1, int acc) {
  const uint32_t m0 = sign_mask4(signs), m1 = sign_mask4(signs >> 4);
  acc = __dp4a((int)__vsub4(g0 ^ m0, m0), (int)x0, acc);
  return __dp4a((int)__vsub4(g1 ^ m1, m1), (int)x1, acc);
}

template <> struct G1<T_IQ2_XS> {   // half d | u16 qs[32] | u8 scales[8]   (vecdotq.cuh:1554-1583)
  static constexpr int UPB = 8, XW = 8, XD = 2, UMAX = 4;
  static __device__ __forceinline__ void load_x(const uint8_t* qs, const float2* ds, int u, int b, uint32_t (&x)[XW], float (&xd)[XD]) {
    G1<T_Q8_0>::load_x(qs, ds, u, b, x, xd);
  }
  static __device__ __forceinline__ float unit(uint32_t blk, int ib, const uint32_t (&x)[XW], const float (&xd)[XD], const Tab1&) {
    const float d = plh(blk);
    uint32_t q[2];
    lds_a2<2>(blk + 2 + 8 * ib, q);
    const uint32_t sc = pl8(blk + 66 + ib);
    int s1 = 0, s2 = 0;
#pragma unroll
    for (int l = 0; l < 4; ++l) {
      const uint32_t idx = (q[l >> 1] >> (16 * (l & 1))) & 0xFFFFu;
      const uint64_t g = __ldg(&d_iq2xs_grid[idx & 511]);
      const int v = dot8_signed((uint32_t)g, (uint32_t)(g >> 32), signs_from7(idx >> 9), x[2 * l], x[2 * l + 1], 0);
      if (l < 2) s1 += v; else s2 += v;
    }
    return d * xd[0] * 0.25f * ((0.5f + (float)(sc & 0xf)) * (float)s1 + (0.5f + (float)(sc >> 4)) * (float)s2);
  }
};

template <> struct G1<T_IQ2_S> {   // half d | u8 qs[32] | u8 signs[32] | u8 qh[8] | u8 scales[8]   (vecdotq.cuh:1585-1620)
  static constexpr int UPB = 8, XW = 8, XD = 2, UMAX = 4;
  static __device__ __forceinline__ void load_x(const uint8_t* qs, const float2* ds, int u, int b, uint32_t (&x)[XW], float (&xd)[XD]) {
    G1<T_Q8_0>::load_x(qs, ds, u, b, x, xd);
  }
  static __device__ __forceinline__ float unit(uint32_t blk, int ib, const uint32_t (&x)[XW], const float (&xd)[XD], const Tab1&) {
    const float d = plh(blk);
    uint32_t q[1], sg[1];
    lds_a2<1>(blk + 2 + 4 * ib, q);
    lds_a2<1>(blk + 34 + 4 * ib, sg);
    const uint32_t qh = pl8(blk + 66 + ib), sc = pl8(blk + 74 + ib);
    int s1 = 0, s2 = 0;
#pragma unroll
    for (int l = 0; l < 4; ++l) {
      const uint64_t g = __ldg(&d_iq2s_grid[((q[0] >> (8 * l)) & 0xFF) | ((qh << (8 - 2 * l)) & 0x300)]);
      const int v = dot8_signed((uint32_t)g, (uint32_t)(g >> 32), (sg[0] >> (8 * l)) & 0xFF, x[2 * l], x[2 * l + 1], 0);
      if (l < 2) s1 += v; else s2 += v;
    }
    return d * xd[0] * 0.25f * ((0.5f + (float)(sc & 0xf)) * (float)s1 + (0.5f + (float)(sc >> 4)) * (float)s2);
  }
};

template <> struct G1<T_IQ3_XXS> {   // half d | u8 qs[64] | u32 scale_and_signs[8]   (vecdotq.cuh:1622-1647)
  static constexpr int UPB = 8, XW = 8, XD = 2, UMAX = 4;
  static __device__ __forceinline__ void load_x(const uint8_t* qs, const float2* ds, int u, int b, uint32_t (&x)[XW], float (&xd)[XD]) {
    G1<T_Q8_0>::load_x(qs, ds, u, b, x, xd);
  }
  static __device__ __forceinline__ float unit(uint32_t blk, int ib, const uint32_t (&x)[XW], const float (&xd)[XD], const Tab1&) {
    const float d = plh(blk);
    uint32_t q[2], a[1];
    lds_a2<2>(blk + 2 + 8 * ib, q);
    lds_a2<1>(blk + 66 + 4 * ib, a);
    const uint32_t aux = a[0];
    int s = 0;
#pragma unroll
    for (int l = 0; l < 4; ++l) {
      const uint32_t w = q[l >> 1] >> (16 * (l & 1));
      const uint32_t g0 = __ldg(&d_iq3xxs_grid[w & 0xFF]), g1 = __ldg(&d_iq3xxs_grid[(w >> 8) & 0xFF]);
      s = dot8_signed(g0, g1, signs_from7((aux >> (7 * l)) & 127), x[2 * l], x[2 * l + 1], s);
    }
    return d * (0.5f + (float)(aux >> 28)) * xd[0] * 0.5f * (float)s;
  }
};

template <> struct G1<T_IQ3_S> {   // half d | u8 qs[64] | u8 qh[8] | u8 signs[32] | u8 scales[4]   (vecdotq.cuh:1649-1672)
  static constexpr int UPB = 8, XW = 8, XD = 2, UMAX = 4;
  static __device__ __forceinline__ void load_x(const uint8_t* qs, const float2* ds, int u, int b, uint32_t (&x)[XW], float (&xd)[XD]) {
    G1<T_Q8_0>::load_x(qs, ds, u, b, x, xd);
  }
  static __device__ __forceinline__ float unit(uint32_t blk, int ib, const uint32_t (&x)[XW], const float (&xd)[XD], const Tab1&) {
    const float d = plh(blk);
    uint32_t q[2], sg[1];
    lds_a2<2>(blk + 2 + 8 * ib, q);
    lds_a2<1>(blk + 74 + 4 * ib, sg);
    const uint32_t qh = pl8(blk + 66 + ib);
    const uint32_t sc = (pl8(blk + 106 + (ib >> 1)) >> (4 * (ib & 1))) & 0xf;
    int s = 0;
#pragma unroll
    for (int l = 0; l < 4; ++l) {
      const uint32_t w = q[l >> 1] >> (16 * (l & 1));
      const uint32_t g0 = __ldg(&d_iq3s_grid[(w & 0xFF) | ((qh << (8 - 2 * l)) & 256)]);
      const uint32_t g1 = __ldg(&d_iq3s_grid[((w >> 8) & 0xFF) | ((qh << (7 - 2 * l)) & 256)]);
      s = dot8_signed(g0, g1, (sg[0] >> (8 * l)) & 0xFF, x[2 * l], x[2 * l + 1], s);
    }
    return d * (0.5f + (float)sc) * xd[0] * 0.5f * (float)s;
  }
};

template <> struct G1<T_IQ1_S> {   // half d | u8 qs[32] | u16 qh[8]   (vecdotq.cuh:1674-1704); xd[1] = fp16 sum of the 32 inputs
  static constexpr int UPB = 8, XW = 8, XD = 2, UMAX = 4;
  static __device__ __forceinline__ void load_x(const uint8_t* qs, const float2* ds, int u, int b, uint32_t (&x)[XW], float (&xd)[XD]) {
    G1<T_Q8_0>::load_x(qs, ds, u, b, x, xd);
  }
  static __device__ __forceinline__ float unit(uint32_t blk, int ib, const uint32_t (&x)[XW], const float (&xd)[XD], const Tab1&) {
    const float d = plh(blk);
    uint32_t q[1];
    lds_a2<1>(blk + 2 + 4 * ib, q);
    const uint32_t qh = pl16(blk + 34 + 2 * ib);
    int s = 0;
#pragma unroll
    for (int l = 0; l < 4; ++l) {
      const uint32_t g = __ldg(&d_iq1s_grid[((q[0] >> (8 * l)) & 0xFF) | (((qh >> (3 * l)) & 7) << 8)]);
      s = __dp4a((int)(g & 0x0F0F0F0Fu), (int)x[2 * l], s);
      s = __dp4a((int)((g >> 4) & 0x0F0F0F0Fu), (int)x[2 * l + 1], s);
    }
    const float delta = (qh & 0x8000u) ? -1.f - 0.125f : -1.f + 0.125f;
    return d * (float)(2 * ((qh >> 12) & 7) + 1) * (xd[0] * (float)s + xd[1] * delta);
  }
};

template <> struct G1<T_IQ1_M> {   // u8 qs[32] | u8 qh[16] | u16 scales[4] (the fp16 scale in their top nibbles)   (vecdotq.cuh:1706-1750)
  static constexpr int UPB = 8, XW = 8, XD = 2, UMAX = 4;
  static __device__ __forceinline__ void load_x(const uint8_t* qs, const float2* ds, int u, int b, uint32_t (&x)[XW], float (&xd)[XD]) {
    G1<T_Q8_0>::load_x(qs, ds, u, b, x, xd);
  }
  static __device__ __forceinline__ float unit(uint32_t blk, int ib, const uint32_t (&x)[XW], const float (&xd)[XD], const Tab1&) {
    const uint32_t q = pl32(blk + 4 * ib);                 // 56-byte blocks: 8-byte aligned
    const uint32_t qh = pl16(blk + 32 + 2 * ib);
    const uint2 scw = pl64(blk + 48);
    const uint32_t s16 = ((scw.x >> 12) & 0x000Fu) | ((scw.x >> 24) & 0x00F0u) | ((scw.y >> 4) & 0x0F00u) | ((scw.y >> 16) & 0xF000u);
    const float d = __half2float(__ushort_as_half((unsigned short)s16));
    float part[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      int si = 0;
      float sf = 0.f;
#pragma unroll
      for (int l2 = 0; l2 < 2; ++l2) {
        const int l = 2 * h + l2;
        const uint32_t qhl = qh >> (4 * l);
        const uint32_t g = __ldg(&d_iq1s_grid[((q >> (8 * l)) & 0xFF) | ((qhl & 7) << 8)]);
        si = __dp4a((int)(g & 0x0F0F0F0Fu), (int)x[2 * l], si);
        si = __dp4a((int)((g >> 4) & 0x0F0F0F0Fu), (int)x[2 * l + 1], si);
        const int sy = __dp4a((int)x[2 * l + 1], 0x01010101, __dp4a((int)x[2 * l], 0x01010101, 0));
        sf += ((qhl & 8u) ? -1.f - 0.125f : -1.f + 0.125f) * (float)sy;
      }
      part[h] = (float)si + sf;
    }
    const uint32_t tmp = (((ib & 4) ? scw.y : scw.x) >> (16 * ((ib >> 1) & 1) + 6 * (ib & 1)));   // scales word ib/2, shifted by 6*(ib%2)
    return d * xd[0] * (part[0] * (float)(2 * (tmp & 7) + 1) + part[1] * (float)(2 * ((tmp >> 3) & 7) + 1));
  }
};

// ---- Q2_K: scales[16] | qs[64] | d | dmin; unit g = 32 values = sub-blocks 2g, 2g+1 (vecdotq.cuh:204-232, 923-944) ----
// value 128n + 32i + l = (qs[32n + l] >> 2i) & 3, so q8_1 block g = 4n + i reads the 32 bytes qs[32n ..] shifted by 2i.
// The min term needs sum(q8) of each 16-value half: constants of the lane, packed in x[8].
template <> struct G1<T_Q2_K> {
  static constexpr int UPB = 8, XW = 9, XD = 2, UMAX = 4;
  static __device__ __forceinline__ void load_x(const uint8_t* qs, const float2* ds, int u, int, uint32_t (&x)[XW], float (&xd)[XD]) {
    const uint4* p = reinterpret_cast<const uint4*>(qs + (size_t)u * 32);
    const uint4 a = p[0], b = p[1];
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
    int s0 = 0, s1 = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      s0 = __dp4a(0x01010101, (int)x[i], s0);
      s1 = __dp4a(0x01010101, (int)x[4 + i], s1);
    }
    x[8] = ((uint32_t)s0 & 0xFFFFu) | ((uint32_t)s1 << 16);
    const float2 d = ds[u];
    xd[0] = d.x; xd[1] = d.y;
  }
  static __device__ __forceinline__ float unit(uint32_t blk, int g, const uint32_t (&x)[XW], const float (&xd)[XD], const Tab1&) {
    const __half2 dm = u32_as_half2(pl32(blk + 80));       // 84-byte blocks: 4-byte aligned
    const uint32_t sc = pl16(blk + 2 * g);
    const uint32_t qb = blk + 16 + 32 * (g >> 2), sh = 2 * (g & 3);
    int a0 = 0, a1 = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      a0 = __dp4a((int)((pl32(qb + 4 * i) >> sh) & 0x03030303u), (int)x[i], a0);
      a1 = __dp4a((int)((pl32(qb + 16 + 4 * i) >> sh) & 0x03030303u), (int)x[4 + i], a1);
    }
    const int s0 = (int)(short)(x[8] & 0xFFFFu), s1 = (int)(short)(x[8] >> 16);
    const float sd = (float)(a0 * (int)(sc & 0xF) + a1 * (int)((sc >> 8) & 0xF));
    const float sm = (float)(s0 * (int)((sc >> 4) & 0xF) + s1 * (int)(sc >> 12));
    return xd[0] * (__low2float(dm) * sd - __high2float(dm) * sm);
  }
};

// ---- Q3_K: hmask[32] | qs[64] | scales[12] | d; unit g = 32 values (vecdotq.cuh:269-300, 1024-1048) ----
// value 128n + 32i + l = ((qs[32n + l] >> 2i) & 3) - (bit 4n+i of hmask[l] ? 0 : 4); 6-bit scales minus 32.
template <> struct G1<T_Q3_K> {
  static constexpr int UPB = 8, XW = 8, XD = 2, UMAX = 4;
  static __device__ __forceinline__ void load_x(const uint8_t* qs, const float2* ds, int u, int b, uint32_t (&x)[XW], float (&xd)[XD]) {
    G1<T_Q8_0>::load_x(qs, ds, u, b, x, xd);
  }
  static __device__ __forceinline__ float unit(uint32_t blk, int g, const uint32_t (&x)[XW], const float (&xd)[XD], const Tab1&) {
    uint32_t hm[8], q[8];
    lds_a2<8>(blk, hm);                                     // 110-byte blocks: 2-byte aligned
    lds_a2<8>(blk + 32 + 32 * (g >> 2), q);
    const uint32_t lo = pl16(blk + 96 + ((2 * g) & 7)) >> (4 * (g >> 2)), hi = pl16(blk + 104 + ((2 * g) & 3)) >> (2 * (g >> 1));
    const int sc0 = (int)((lo & 0xF) | ((hi & 3) << 4)) - 32, sc1 = (int)(((lo >> 8) & 0xF) | (((hi >> 8) & 3) << 4)) - 32;
    const uint32_t sh = 2 * (g & 3);
    int a0 = 0, a1 = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t v = __vsub4((q[i] >> sh) & 0x03030303u, ((~hm[i] >> g) << 2) & 0x04040404u);
      if (i < 4) a0 = __dp4a((int)v, (int)x[i], a0);
      else a1 = __dp4a((int)v, (int)x[i], a1);
    }
    return plh(blk + 108) * xd[0] * (float)(a0 * sc0 + a1 * sc1);
  }
};

// ---- Q4_1: value = q*d + m; the min term uses the fp16 sum of the inputs (vecdotq.cuh:72-96) -----
// Both products of the reference (d*d8 and m*s8) are formed in half precision (__hmul2) before
// they are widened; the same is done here.
__device__ __forceinline__ float hmul_f32(float a, float b) {   // a, b hold fp16 values: their product rounded to fp16
  return __half2float(__hmul(__float2half_rn(a), __float2half_rn(b)));
}
template <> struct G1<T_Q4_1> {
  static constexpr int UPB = 1, XW = 8, XD = 2, UMAX = 4;
  static __device__ __forceinline__ void load_x(const uint8_t* qs, const float2* ds, int u, int b, uint32_t (&x)[XW], float (&xd)[XD]) {
    G1<T_Q8_0>::load_x(qs, ds, u, b, x, xd);
  }
  static __device__ __forceinline__ float unit(uint32_t blk, int, const uint32_t (&x)[XW], const float (&xd)[XD], const Tab1&) {
    const __half2 dm = u32_as_half2(pl32(blk));            // 20-byte blocks: 4-byte aligned
    int lo = 0, hi = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t q = pl32(blk + 4 + 4 * i);
      lo = dp4a_us1(q & 0x0F0F0F0Fu, x[i], lo);
      hi = dp4a_us1(q & 0xF0F0F0F0u, x[4 + i], hi);
    }
    return (float)(lo + (hi >> 4)) * hmul_f32(__low2float(dm), xd[0]) + hmul_f32(__high2float(dm), xd[1]);
  }
};

// fifth bits of four values (bits 0..3 of x) moved to bit 4 of the four bytes of a word: the
// multiplier puts bit k at 8k + 4 and all sixteen partial products fall on different bit positions
__device__ __forceinline__ uint32_t spread_bit4(uint32_t x) { return ((x & 0xFu) * 0x02040810u) & 0x10101010u; }

// ---- Q5_0: value = (q - 16)*d, q = 4 low bits | fifth bit from qh (vecdotq.cuh:101-129) ------------
template <> struct G1<T_Q5_0> {
  static constexpr int UPB = 1, XW = 8, XD = 2, UMAX = 4;
  static __device__ __forceinline__ void load_x(const uint8_t* qs, const float2* ds, int u, int b, uint32_t (&x)[XW], float (&xd)[XD]) {
    G1<T_Q8_0>::load_x(qs, ds, u, b, x, xd);
  }
  static __device__ __forceinline__ float unit(uint32_t blk, int, const uint32_t (&x)[XW], const float (&xd)[XD], const Tab1&) {
    const float d = plh(blk);
    uint32_t w[5];
    lds_a2<5>(blk + 2, w);                                    // qh, then 16 bytes of nibbles (2-byte aligned)
    const uint32_t qh = w[0];
    int s0 = 0, s1 = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      s0 = dp4a_us1((w[1 + i] & 0x0F0F0F0Fu) | spread_bit4(qh >> (4 * i)), x[i], s0);
      s1 = dp4a_us1(((w[1 + i] >> 4) & 0x0F0F0F0Fu) | spread_bit4(qh >> (16 + 4 * i)), x[4 + i], s1);
    }
    return d * ((float)(s0 + s1) * xd[0] - 16.0f * xd[1]);
  }
};

// ---- Q5_1: value = q*d + m (vecdotq.cuh:134-163) -------------------------------------------------
template <> struct G1<T_Q5_1> {
  static constexpr int UPB = 1, XW = 8, XD = 2, UMAX = 4;
  static __device__ __forceinline__ void load_x(const uint8_t* qs, const float2* ds, int u, int b, uint32_t (&x)[XW], float (&xd)[XD]) {
    G1<T_Q8_0>::load_x(qs, ds, u, b, x, xd);
  }
  static __device__ __forceinline__ float unit(uint32_t blk, int, const uint32_t (&x)[XW], const float (&xd)[XD], const Tab1&) {
    const uint2 hdr = pl64(blk);                             // 24-byte blocks: 8-byte aligned
    const __half2 dm = u32_as_half2(hdr.x);
    const uint32_t qh = hdr.y;
    const uint2 qa = pl64(blk + 8), qb = pl64(blk + 16);
    const uint32_t w[4] = {qa.x, qa.y, qb.x, qb.y};
    int s0 = 0, s1 = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      s0 = dp4a_us1((w[i] & 0x0F0F0F0Fu) | spread_bit4(qh >> (4 * i)), x[i], s0);
      s1 = dp4a_us1(((w[i] >> 4) & 0x0F0F0F0Fu) | spread_bit4(qh >> (16 + 4 * i)), x[4 + i], s1);
    }
    return (float)(s0 + s1) * hmul_f32(__low2float(dm), xd[0]) + hmul_f32(__high2float(dm), xd[1]);
  }
};

// ---- IQ4_NL: 32 values, levels from the IQ4 table (vecdotq.cuh:1766-1789); see G1<T_IQ4_XS> -------
template <> struct G1<T_IQ4_NL> {
  static constexpr int UPB = 1, XW = 8, XD = 2, UMAX = 4;
  static __device__ __forceinline__ void load_x(const uint8_t* qs, const float2* ds, int u, int b, uint32_t (&x)[XW], float (&xd)[XD]) {
    G1<T_IQ4_XS>::load_x(qs, ds, u, b, x, xd);
  }
  static __device__ __forceinline__ float unit(uint32_t blk, int, const uint32_t (&x)[XW], const float (&xd)[XD], const Tab1& t) {
    const float d = plh(blk);
    uint32_t q[4];
    lds_a2<4>(blk + 2, q);
    int s0 = 0, s1 = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t q3 = q[i] & 0x77777777u;
      const uint32_t sel = ((q[i] & 0x88888888u) >> 1) | 0x32103210u;
      s0 = __dp4a((int)G1<T_IQ4_XS>::lut4(q3, sel, t), (int)x[2 * i], s0);
      s1 = __dp4a((int)G1<T_IQ4_XS>::lut4(q3 >> 16, sel >> 16, t), (int)x[2 * i + 1], s1);
    }
    return d * xd[0] * (float)(s0 + s1);
  }
};

// ---- Q5_K: like Q4_K with a fifth bit from qh; unit p = 64 values (sub-blocks 2p, 2p+1) ------------
// (vecdotq.cuh:386-413, 1279-1323; the min term uses d8 * sum(q8), as for Q4_K)
template <> struct G1<T_Q5_K> {
  static constexpr int UPB = 4, XW = 16, XD = 4, UMAX = 2;
  static __device__ __forceinline__ void load_x(const uint8_t* qs, const float2* ds, int u, int b, uint32_t (&x)[XW], float (&xd)[XD]) {
    G1<T_Q4_K>::load_x(qs, ds, u, b, x, xd);
  }
  static __device__ __forceinline__ float unit(uint32_t blk, int p, const uint32_t (&x)[XW], const float (&xd)[XD], const Tab1&) {
    const uint4 hdr = pl128(blk);
    const __half2 dm = u32_as_half2(hdr.x);
    const float d = __low2float(dm), dmin = __high2float(dm);
    const int sh = 16 * (p & 1);
    const uint32_t a = hdr.y >> sh, b = hdr.z >> sh, c = hdr.w >> sh;
    // get_scale_min_k4: both cases computed and merged with a mask (lanes of a warp differ in p:
    // a branch here would run both sides one after the other)
    const uint32_t lowm = p < 2 ? 0xFFFFFFFFu : 0u;
    const uint32_t sc2 = ((a & 0x3F3Fu) & lowm) | (((c & 0x0F0Fu) | ((a >> 2) & 0x3030u)) & ~lowm);
    const uint32_t mn2 = ((b & 0x3F3Fu) & lowm) | ((((c >> 4) & 0x0F0Fu) | ((b >> 2) & 0x3030u)) & ~lowm);
    const int sc0 = sc2 & 0xFF, sc1 = (sc2 >> 8) & 0xFF;
    const float m0 = (float)(mn2 & 0xFF), m1 = (float)((mn2 >> 8) & 0xFF);
    const uint4 ha = pl128(blk + 16), hb = pl128(blk + 32);                 // qh[0..31]: bit 2p / 2p+1 of byte l
    const uint4 qa = pl128(blk + 48 + 32 * p), qb = pl128(blk + 64 + 32 * p);
    const uint32_t q[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
    const uint32_t h[8] = {ha.x, ha.y, ha.z, ha.w, hb.x, hb.y, hb.z, hb.w};
    int a0 = 0, a1 = 0, b0 = 0, b1 = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const uint32_t hh = h[2 * i + e] >> (2 * p);
        const uint32_t lo = (q[2 * i + e] & 0x0F0F0F0Fu) | ((hh << 4) & 0x10101010u);
        const uint32_t hi = ((q[2 * i + e] >> 4) & 0x0F0F0F0Fu) | ((hh << 3) & 0x10101010u);
        if (e == 0) {
          a0 = dp4a_us1(lo, x[2 * i], a0);
          b0 = dp4a_us1(hi, x[8 + 2 * i], b0);
        } else {
          a1 = dp4a_us1(lo, x[2 * i + 1], a1);
          b1 = dp4a_us1(hi, x[8 + 2 * i + 1], b1);
        }
      }
    }
    return d * (xd[0] * (float)((a0 + a1) * sc0) + xd[2] * (float)((b0 + b1) * sc1)) - dmin * (xd[1] * m0 + xd[3] * m1);
  }
};

// ---- kernel ---------------------------------------------------------------------------------
//
// Work item of a warp = a group of up to G1_R consecutive rows (x its K-slice).  With one slice
// the rows of a group are contiguous in memory and arrive with ONE bulk copy; with several
// slices each row's slice is its own copy into a padded slot of the stage.  Grouping rows
// amortises the per-item costs (copy issue, barrier wait, address arithmetic) over G1_R rows.
//
// Rows are shared out over the grid's "row lanes" (a row lane = the ks warps of a CTA that work
// on the same rows; rl lanes per CTA): lane w owns the contiguous rows [w*q + min(w, r), ...) with
// q = N / lanes, r = N % lanes -- every lane gets q or q+1 rows, so no lane runs a whole extra
// pass, a lane streams one contiguous byte range, and the rows of a CTA are one contiguous range.
// (Dealing row groups to the lanes in turn measured the same with one slice and 4 % slower with
// K-slices; giving a lane a smaller FIRST item, to start its arithmetic sooner, was slower on every
// shape -- one more barrier round trip per warp costs more than the earlier start gains.)

constexpr int G1_R = 4;
constexpr int G1_MAX_WORLD = 8;

struct G1Params {
  const uint8_t* w;
  int64_t w_bytes;
  const uint8_t* xq;     // SoA q8_1 of the vector: int8 qs[kpad] then float2 ds[kpad/32]
  void* y;
  int64_t n, k;
  int bpr;               // blocks per row
  int ks, rl;            // K-slices per row, row lanes per CTA (ks * rl <= 8)
  int slice_q, slice_r;  // slice i holds slice_q + (i < slice_r) blocks, so no slice is ever empty
  int rows_per_item;     // <= G1_R
  int slot_bytes;        // distance between the rows of an item inside a stage
  int stages, stage_bytes;
  int partial_bytes;     // shared memory for the staged results (0 when every warp stores its own)
  // Activations not yet quantized (x_raw != null): xq is unused; every CTA quantizes the MV vectors it
  // needs (K values each, element type = the output type) to q8_1 in its own shared memory right after
  // the programmatic wait -- bit-identical to the standalone quantizer -- so a decode GEMV is ONE launch.
  const void* x_raw;
  int x_sum_mode;        // 1: the {d, sum} pair holds d * sum(q) instead of the fp16 sum of the inputs
  int x_bytes;           // shared memory for the quantized activations (0 with x_alias)
  int x_alias;           // 1: they sit in the LAST stage of warp 0's ring, which is filled only after every warp has
                         //    its activations in registers (the first stages - 1 are on their way before)
  int ks_shift;          // log2(ks)
  int q_rows, r_rows;    // N / lanes and N % lanes for lanes = grid.x * rl
  unsigned inv_r;        // ceil(2^32 / rows_per_item): x / rows_per_item = umulhi(x, inv_r)  (unused when it is 1)
  int* status;
  // MoE decode (topk_ids != null, one vector): blockIdx.y is an output row s of y; it uses the
  // weights of expert topk_ids[s] (experts back to back, expert_bytes apart) and the activation
  // vector s / top_k of the xq_vecs quantized ones
  const int32_t* topk_ids;
  int top_k, n_experts, xq_vecs, moe_slots;
  int vec0;              // dense: first of the MV vectors this launch handles, out of the xq_vecs in the scratch
  int64_t expert_bytes;
  // Tensor-parallel output (world > 0): every result is sent to ALL ranks (this one included) as
  // a packet {value, tag} written with one store into ll_peer[r][y_off + row]; tag = epoch[slot],
  // this launch's number, which the activation quantizer queued just before this kernel has
  // already incremented.  A reader that finds the tag it expects has the value: no fence, no flag.
  int world, slot;
  const unsigned* epoch;
  int64_t y_off;
  void* ll_peer[G1_MAX_WORLD];
};

template <typename out_t>
__device__ __forceinline__ void store_result(const G1Params& p, int64_t row, float v, int m, unsigned tag) {
  if (p.world == 0) {
    m = p.topk_ids ? (int)blockIdx.y : m + p.vec0;   // MoE decode: one output row of y per (token, expert) pair
    static_cast<out_t*>(p.y)[(int64_t)m * p.n + row] = from_float<out_t>(v);
    return;
  }
  const out_t o = from_float<out_t>(v);
  if (sizeof(out_t) == 2) {
    const uint32_t pk = (uint32_t)(*reinterpret_cast<const uint16_t*>(&o)) | (tag << 16);
#pragma unroll 1
    for (int r = 0; r < p.world; ++r) {
      uint32_t* dst = static_cast<uint32_t*>(p.ll_peer[r]) + p.y_off + row;
      asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(dst), "r"(pk) : "memory");
    }
  } else {
    const unsigned long long pk = (unsigned long long)(*reinterpret_cast<const uint32_t*>(&o)) | ((unsigned long long)tag << 32);
#pragma unroll 1
    for (int r = 0; r < p.world; ++r) {
      unsigned long long* dst = static_cast<unsigned long long*>(p.ll_peer[r]) + p.y_off + row;
      asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst), "l"(pk) : "memory");
    }
  }
}

// MV activation vectors share one pass over the weights (MV = 1 or 2): a lane keeps the
// activations of MV vectors for UMAX / MV units, so rows are cut into MV times as many K-slices
// and the register budget stays that of one vector.
template <int TYPE, typename out_t, int MV>
__global__ void __launch_bounds__(G1_WARPS * 32, 2) gemv1_kernel(const G1Params p) {
  extern __shared__ __align__(128) uint8_t smem[];
  using T = G1<TYPE>;
  static_assert(T::UMAX % MV == 0, "units per lane must divide by the vector count");
  constexpr int TS = BlockTraits<TYPE>::TS, UPB = T::UPB, UMAX = T::UMAX / MV;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kpad = (int)round_up(p.k, 512);
  const uint8_t* wb = p.w;      // this CTA's weight matrix
  int vec0 = p.vec0;            // its first activation vector
  if (p.topk_ids) {
    const int e = p.topk_ids[blockIdx.y];
    if (e < 0 || e >= p.n_experts) return;   // not a valid expert: the row is left as it is
    wb += (int64_t)e * p.expert_bytes;
    vec0 = (int)blockIdx.y / p.top_k;
  }

  uint8_t* cur = smem;
  Tab1 tb;
  tb.grid = 0;
  tb.smask = 0;
  if (TYPE == T_IQ2_XXS) {
    // Both code books are stored G1_TAB_COPIES times, copy c in the 8-byte column c of every
    // 128-byte line: lane l reads copy l % 16, and since a 64-bit shared load is served one
    // half-warp at a time, the 16 lanes of a half-warp hit 16 different bank pairs whatever
    // entries they ask for.  (One copy costs a 3- to 4-way bank conflict on almost every look-up:
    // 32 unrelated 8-byte entries per load.  Eight copies -- half the shared memory, room for larger
    // work items -- measured slower: 28672x8192 36.7 us against 29.5 us with sixteen.)
    uint2* g = reinterpret_cast<uint2*>(cur);
    uint2* sm = g + 256 * G1_TAB_COPIES;
    cur += (256 + 128) * 8 * G1_TAB_COPIES;
    tb.grid = smem_u32(g + (lane & (G1_TAB_COPIES - 1)));
    tb.smask = smem_u32(sm + (lane & (G1_TAB_COPIES - 1)));
  }
  if (TYPE == T_IQ4_XS || TYPE == T_IQ4_NL) {
    const uint32_t* kv = reinterpret_cast<const uint32_t*>(d_kvalues_iq4nl);
#pragma unroll
    for (int i = 0; i < 4; ++i) tb.kv[i] = kv[i];
  }
  uint8_t* s_x = cur;                               // quantized activations (when this kernel quantizes them itself)
  cur += p.x_bytes;
  float* partial = reinterpret_cast<float*>(cur);  // [rl][G1_BATCH][G1_R][MV][ks], present only when results are staged
  cur += p.partial_bytes;
  if (p.x_alias) s_x = cur + (size_t)(p.stages - 1) * p.stage_bytes;
  uint8_t* ring = cur + (size_t)warp * p.stages * p.stage_bytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(cur + (size_t)G1_WARPS * p.stages * p.stage_bytes) + warp * p.stages;
  if (lane == 0)
    for (int s = 0; s < p.stages; ++s) mbar_init(&bars[s], 1);
  fence_barrier_init();
  __syncwarp();

  // (everything below is 32-bit arithmetic on values the host prepared: a 64-bit division per warp
  //  costs as much as half a row of dot products, and a warp only has six or seven rows)
  const bool active = warp < p.ks * p.rl;
  const int ks_i = warp & (p.ks - 1), rl_i = warp >> p.ks_shift;
  const int sb0 = ks_i * p.slice_q + min(ks_i, p.slice_r);
  const int nblk = active ? p.slice_q + (ks_i < p.slice_r ? 1 : 0) : 0;
  const int units = nblk * UPB;
  const int R = p.rows_per_item;
  const int64_t row_bytes = (int64_t)p.bpr * TS;
  const int64_t w_safe = p.w_bytes & ~int64_t(15);
  const uint32_t slice_bytes = (uint32_t)nblk * TS;
  const bool contiguous = p.ks == 1;
  const bool staged = p.ks > 1 || p.world > 0;   // results meet in shared memory before they are stored

  // ---- which rows: row lane wl (= the ks warps of a CTA that work on the same rows) owns the
  // contiguous range [wl * q + min(wl, r), ...) of q or q + 1 rows, q = N / lanes, r = N % lanes ----
  auto lane_row0 = [&](int l) -> int {
    const int wl = (int)blockIdx.x * p.rl + l;
    return wl * p.q_rows + min(wl, p.r_rows);
  };
  auto lane_rows = [&](int l) -> int { return p.q_rows + (((int)blockIdx.x * p.rl + l) < p.r_rows ? 1 : 0); };
  // first row and row count of item i of row lane l
  auto item = [&](int l, int i, int& row, int& cnt) {
    const int done = i * R;
    row = lane_row0(l) + done;
    cnt = min(R, max(lane_rows(l) - done, 0));
  };
  auto lane_iters = [&](int l) -> int {
    const unsigned x = (unsigned)(lane_rows(l) + R - 1);
    return (int)(R == 1 ? x : __umulhi(x, p.inv_r));   // x / R
  };
  const int iters = lane_iters(0);   // lane 0 of a CTA never has fewer passes than the others: uniform over the CTA
  const int my_iters = (active && nblk > 0) ? lane_iters(rl_i) : 0;

  // copy of the rows [r0, r0 + cnt) (this warp's slice of them) into stage st
  auto issue = [&](int r0, int cnt, int st) {
    uint8_t* dst = ring + (size_t)st * p.stage_bytes;
    if (contiguous) {
      if (lane == 0) {
        const int64_t beg = (int64_t)r0 * row_bytes, end = beg + (int64_t)cnt * row_bytes;
        const int64_t abeg = beg & ~int64_t(15);
        int64_t aend = (end + 15) & ~int64_t(15);
        if (aend > w_safe) aend = w_safe;
        const uint32_t bytes = aend > abeg ? (uint32_t)(aend - abeg) : 0u;
        if (bytes) {
          mbar_expect_tx(&bars[st], bytes);
          bulk_g2s(dst, wb + abeg, bytes, &bars[st]);
        } else {
          mbar_arrive(&bars[st]);
        }
      }
    } else {
      // one copy per row; lane j computes and issues row j's, lane 0 announces the byte total first
      const int64_t beg = (int64_t)(r0 + lane) * row_bytes + (int64_t)sb0 * TS, end = beg + slice_bytes;
      const int64_t abeg = beg & ~int64_t(15);
      int64_t aend = (end + 15) & ~int64_t(15);
      if (aend > w_safe) aend = w_safe;
      const uint32_t bytes = (lane < cnt && aend > abeg) ? (uint32_t)(aend - abeg) : 0u;
      uint32_t total = bytes;
#pragma unroll
      for (int m = 1; m < G1_R; m <<= 1) total += __shfl_xor_sync(0xffffffffu, total, m);  // lanes 0..3 hold the sum of lanes 0..3
      if (lane == 0) {
        if (total) mbar_expect_tx(&bars[st], total);
        else mbar_arrive(&bars[st]);
      }
      __syncwarp();
      if (bytes) bulk_g2s(dst + (size_t)lane * p.slot_bytes, wb + abeg, bytes, &bars[st]);
    }
  };

  // All stages but one are filled before anything else happens, while the previous kernel of the
  // stream is still draining and before the activations exist; the last one follows when the
  // activations are in registers.  (Filling every stage at once was slower: the memory system
  // serves what is outstanding interleaved, so every warp's FIRST item arrived later and the first
  // dot products with it -- 14336x4096 Q4_K 8.6 us against 8.0 us.)
  int p_it = 0, p_st = 0;
  for (int s = 0; s < p.stages - 1; ++s) {
    if (p_it < my_iters) {
      int r0, cnt;
      item(rl_i, p_it, r0, cnt);
      issue(r0, cnt, p_st);
      ++p_it;
      if (++p_st == p.stages) p_st = 0;
    }
  }

  if (TYPE == T_IQ2_XXS) {   // fill the code-book copies while the first weight copies are in flight
    uint2* tab_g = reinterpret_cast<uint2*>(smem);
    uint2* tab_s = tab_g + 256 * G1_TAB_COPIES;
    for (int i = threadIdx.x; i < 256 * G1_TAB_COPIES; i += blockDim.x) {
      const uint64_t v = d_iq2xxs_grid[i / G1_TAB_COPIES];
      tab_g[i] = make_uint2((uint32_t)v, (uint32_t)(v >> 32));
    }
    for (int i = threadIdx.x; i < 128 * G1_TAB_COPIES; i += blockDim.x) {
      const uint32_t s = d_ksigns_iq2xs[i / G1_TAB_COPIES];
      uint32_t lo = 0, hi = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        lo |= ((s >> j) & 1u) ? (0xFFu << (8 * j)) : 0u;
        hi |= ((s >> (4 + j)) & 1u) ? (0xFFu << (8 * j)) : 0u;
      }
      tab_s[i] = make_uint2(lo, hi);
    }
  }
  // The weight copies above touch nothing another kernel writes; everything below does.
  pdl_wait();
  const unsigned tag = p.world > 0 ? (sizeof(out_t) == 2 ? (p.epoch[p.slot] & 0xFFFFu) : p.epoch[p.slot]) : 0u;
  // this lane's units (block offset inside the slice, sub-unit) and their activations
  uint32_t xq[MV][UMAX][T::XW];
  float xd[MV][UMAX][T::XD];
  int uoff[UMAX], usub[UMAX];
  const uint8_t* xq_base = p.xq;   // SoA q8_1: int8 codes [vectors][kpad], then float2 {d, sum} [vectors][kpad / 32]
  int xq_vecs = p.xq_vecs, xq_v0 = vec0;
  if (p.x_raw) {
    // Quantize this CTA's MV vectors into shared memory, eight values per thread (four lanes own a
    // block of 32).  The reference's butterfly adds element i to element i^16, then i^8, i^4, i^2,
    // i^1; with lane t of a quad holding elements 8t..8t+7 the first two levels are shuffles across
    // the quad and the last three are adds inside the thread, in the same order, so the fp32 sum (and
    // with it every bit of the result) is that of the standalone quantizer.
    const out_t* xr = static_cast<const out_t*>(p.x_raw) + (size_t)vec0 * p.k;
    const int per_vec = kpad / 8, t = lane & 3;
    float2* s_ds = reinterpret_cast<float2*>(s_x + (size_t)MV * kpad);
    const bool vec_ok = (p.k % 8 == 0) && ((reinterpret_cast<uintptr_t>(xr) & 15) == 0);
    for (int i0 = threadIdx.x; i0 < MV * per_vec; i0 += G1_WARPS * 32) {   // (a multiple of 64 items: whole warps)
      const int v = MV == 1 ? 0 : i0 / per_vec, idx = i0 - v * per_vec, k = idx * 8;
      const out_t* src = xr + (size_t)v * p.k + k;
      float val[8];
      if (vec_ok && k + 8 <= p.k) {
        if (sizeof(out_t) == 4) {
          const float4 a = *reinterpret_cast<const float4*>(src), c = *reinterpret_cast<const float4*>(src + 4);
          val[0] = a.x; val[1] = a.y; val[2] = a.z; val[3] = a.w; val[4] = c.x; val[5] = c.y; val[6] = c.z; val[7] = c.w;
        } else {
          const uint4 a = *reinterpret_cast<const uint4*>(src);
          const out_t* e = reinterpret_cast<const out_t*>(&a);
#pragma unroll
          for (int j = 0; j < 8; ++j) val[j] = to_float<out_t>(e[j]);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) val[j] = k + j < p.k ? to_float<out_t>(src[j]) : 0.0f;
      }
      float amax = 0.f, sm[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        amax = fmaxf(amax, fabsf(val[j]));
        sm[j] = val[j] + __shfl_xor_sync(0xffffffffu, val[j], 2, 32);          // i ^ 16
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
      uint32_t w0 = 0, w1 = 0;
      int qsum = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int8_t qq = amax == 0.0f ? 0 : roundf(val[j] / d);
        qsum += qq;
        if (j < 4) w0 |= ((uint32_t)qq & 0xFFu) << (8 * j);
        else w1 |= ((uint32_t)qq & 0xFFu) << (8 * (j - 4));
      }
      *reinterpret_cast<uint2*>(s_x + (size_t)v * kpad + k) = make_uint2(w0, w1);
      qsum += __shfl_xor_sync(0xffffffffu, qsum, 2, 32);
      qsum += __shfl_xor_sync(0xffffffffu, qsum, 1, 32);
      if (t == 0) {
        const float d8 = __half2float(__float2half(d));
        s_ds[(size_t)v * (kpad / 32) + (k >> 5)] = make_float2(d8, p.x_sum_mode ? d8 * (float)qsum : __half2float(__float2half(sum)));
      }
    }
    __syncthreads();
    xq_base = s_x;
    xq_vecs = MV;
    xq_v0 = 0;
  }
#pragma unroll
  for (int m = 0; m < MV; ++m) {
    const uint8_t* qs = xq_base + (size_t)(xq_v0 + m) * kpad;
    const float2* ds = reinterpret_cast<const float2*>(xq_base + (size_t)xq_vecs * kpad) + (size_t)(xq_v0 + m) * (kpad / 32);
#pragma unroll
    for (int j = 0; j < UMAX; ++j) {
      const int u = lane + 32 * j;
      uoff[j] = (u / UPB) * TS;
      usub[j] = u % UPB;
      if (u < units) {
        T::load_x(qs, ds, sb0 * UPB + u, 0, xq[m][j], xd[m][j]);
      } else {
        // no such unit in this slice: zero activations against the slice's first block, so that the
        // loop below needs no test per unit (it adds d * 0 of a block the row contains anyway)
        uoff[j] = 0;
        usub[j] = 0;
#pragma unroll
        for (int i = 0; i < T::XW; ++i) xq[m][j][i] = 0;
#pragma unroll
        for (int i = 0; i < T::XD; ++i) xd[m][j][i] = 0.f;
      }
    }
  }
  if (TYPE == T_IQ2_XXS) __syncthreads();  // tables staged
  if (p.x_alias) {   // every warp has read its activations: the stage they sat in may now take weights
    __syncthreads();
    fence_proxy_async();
  }
  pdl_trigger();  // activations are in registers: the next kernel may be scheduled behind this one

  int c_st = 0;
  uint32_t c_phase = 0;
  bool dead = false;
  for (int i = 0; i < iters; ++i) {
    const bool mine = i < my_iters && !dead;
    if (mine) {
      if (p_it < my_iters) {   // the stage freed by the previous pass takes the next item
        int r0, cnt2;
        item(rl_i, p_it, r0, cnt2);
        issue(r0, cnt2, p_st);
        ++p_it;
        if (++p_st == p.stages) p_st = 0;
      }
      if (!mbar_wait_bounded(&bars[c_st], c_phase)) {
        if (lane == 0) atomicExch(p.status, E_TIMEOUT);
        dead = true;
      }
    }
    if (mine && !dead) {
      int c_row, cnt;
      item(rl_i, i, c_row, cnt);
      uint8_t* stage = ring + (size_t)c_st * p.stage_bytes;
      const int64_t beg0 = (int64_t)c_row * row_bytes + (int64_t)sb0 * TS;
      const int64_t last_end = beg0 + (int64_t)(cnt - 1) * row_bytes + slice_bytes;
      if (last_end > w_safe) {  // tail bytes the bulk copy must not touch: fetched with plain loads
        const int64_t lbeg = contiguous ? beg0 : last_end - slice_bytes;
        const int64_t abeg = lbeg & ~int64_t(15);
        uint8_t* base = contiguous ? stage : stage + (size_t)(cnt - 1) * p.slot_bytes;
        for (int64_t o = w_safe + lane; o < last_end; o += 32) base[o - abeg] = wb[o];
        __syncwarp();
      }
      const uint32_t stage_s = fresh_stage(smem_u32(stage));   // after the wait and the tail bytes: see pl32
      float acc[MV][G1_R];
#pragma unroll
      for (int rr = 0; rr < G1_R; ++rr)
#pragma unroll
        for (int m = 0; m < MV; ++m) acc[m][rr] = 0.f;
      auto row_data = [&](int rr) -> uint32_t {
        return stage_s + (contiguous ? (uint32_t)(beg0 & 15) + (uint32_t)rr * (uint32_t)row_bytes
                                     : (uint32_t)rr * (uint32_t)p.slot_bytes + (uint32_t)((beg0 + rr * row_bytes) & 15));
      };
      // straight-line code for every row count, so that the loads and the dot-product chains of all
      // cnt * UMAX units can overlap
      auto rows = [&](auto cnt_c) {
        constexpr int C = decltype(cnt_c)::value;
        uint32_t d[C];
#pragma unroll
        for (int rr = 0; rr < C; ++rr) d[rr] = row_data(rr);
        // (the vectors innermost: their two dot products share one set of loads and one header decode)
#pragma unroll
        for (int j = 0; j < UMAX; ++j)
#pragma unroll
          for (int rr = 0; rr < C; ++rr)
#pragma unroll
            for (int m = 0; m < MV; ++m) acc[m][rr] += T::unit(d[rr] + uoff[j], usub[j], xq[m][j], xd[m][j], tb);
      };
      switch (cnt) {
        case 1: rows(std::integral_constant<int, 1>{}); break;
        case 2: rows(std::integral_constant<int, 2>{}); break;
        case 3: rows(std::integral_constant<int, 3>{}); break;
        default: rows(std::integral_constant<int, 4>{}); break;
      }
      // Warp reduction of the cnt row sums together.  The butterfly of ONE value adds lane l^16,
      // then l^8, l^4, l^2, l^1.  With two or four values the first one or two levels are done
      // "transposed": a lane keeps the value of the row its bit 4 (and bit 3) selects and gives the
      // other one away, so that after them every lane holds a partial sum of ONE row and the
      // remaining levels serve all rows at once -- 5 or 6 shuffles instead of 10 to 20.  Every
      // addition has the same two operands as in the one-value butterfly, so the bits of a row's
      // sum do not depend on how many rows shared the item.
#pragma unroll
      for (int m = 0; m < MV; ++m) {
        float v;
        int my_rr;
        if (cnt == 1) {
          v = acc[m][0];
          v += __shfl_xor_sync(0xffffffffu, v, 16);
          v += __shfl_xor_sync(0xffffffffu, v, 8);
          my_rr = 0;
        } else {
          const bool up = (lane & 16) != 0;
          float a = up ? acc[m][1] : acc[m][0];
          a += __shfl_xor_sync(0xffffffffu, up ? acc[m][0] : acc[m][1], 16);
          if (cnt == 2) {
            v = a + __shfl_xor_sync(0xffffffffu, a, 8);
            my_rr = up ? 1 : 0;
          } else {
            float b = up ? acc[m][3] : acc[m][2];
            b += __shfl_xor_sync(0xffffffffu, up ? acc[m][2] : acc[m][3], 16);
            const bool hi = (lane & 8) != 0;
            v = (hi ? b : a) + __shfl_xor_sync(0xffffffffu, hi ? a : b, 8);
            my_rr = (up ? 1 : 0) + (hi ? 2 : 0);
          }
        }
        v += __shfl_xor_sync(0xffffffffu, v, 4);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        if ((lane & 7) == 0 && my_rr < cnt && (cnt > 2 || (lane & 8) == 0) && (cnt > 1 || lane == 0)) {   // one writer lane per row
          if (!staged) store_result<out_t>(p, c_row + my_rr, v, m, 0u);
          else partial[(((rl_i * G1_BATCH + (i % G1_BATCH)) * G1_R + my_rr) * MV + m) * p.ks + ks_i] = v;
        }
      }
      __syncwarp();   // every lane is done with the stage: the next pass may refill it
      if (++c_st == p.stages) { c_st = 0; c_phase ^= 1u; }
    }
    if (staged && ((i % G1_BATCH) == G1_BATCH - 1 || i == iters - 1)) {
      // add the slice partials in slice order and store; every warp of the CTA takes part.
      // Consecutive threads take consecutive rows of one row lane, so the stores (and the
      // packets sent to the other GPUs) leave as runs of adjacent addresses.
      __syncthreads();
      const int i0 = i - (i % G1_BATCH);
      const int per_lane = (i - i0 + 1) * G1_R;
      const int cnt = per_lane * p.rl * MV;
      for (int t = threadIdx.x; t < cnt; t += blockDim.x) {
        const int m = t / (per_lane * p.rl), t2 = t - m * per_lane * p.rl;
        const int gl = t2 / per_lane, t3 = t2 - gl * per_lane;
        const int ii = i0 + t3 / G1_R, rr = t3 % G1_R;
        int r0, c;
        item(gl, ii, r0, c);
        if (rr < c) {
          float s = 0.f;
          for (int q = 0; q < p.ks; ++q) s += partial[(((gl * G1_BATCH + (ii % G1_BATCH)) * G1_R + rr) * MV + m) * p.ks + q];
          store_result<out_t>(p, r0 + rr, s, m, tag);
        }
      }
      __syncthreads();
    }
  }
  if (dead) drain_pause();   // copies this warp still has in flight land before its CTA can retire
}

// ---- host -----------------------------------------------------------------------------------

static int g1_env(const char* name, int dflt) {
  const char* v = getenv(name);
  return v && *v ? atoi(v) : dflt;
}

template <int TYPE, typename out_t, int MV>
static int launch_g1(G1Params p, cudaStream_t stream) {
  using T = G1<TYPE>;
  constexpr int TS = BlockTraits<TYPE>::TS;
  // Two stages per warp measured best on every shape: with three or more (up to the warp's whole
  // share) all of a small matrix is requested at once, the memory system serves the requests
  // interleaved, and every warp's FIRST item arrives late (14336x4096 Q4_K: 9.7 us with 2 stages,
  // 11.1 with 3, 12.9 with 6).
  static const int stages_env = g1_env("GGUF_B200_GEMV1_STAGES", 2);
  static const int ctas_env = g1_env("GGUF_B200_GEMV1_CTAS", 2);
  static const int rows_env = g1_env("GGUF_B200_GEMV1_ROWS", G1_R);
  static const int item_env = g1_env("GGUF_B200_GEMV1_ITEM_BYTES", 7168);
  const int cap_blocks = 32 * (T::UMAX / MV) / T::UPB;  // blocks whose units fit one lane-register set
  int ks = 1;
  while (ks < 8 && (p.bpr + ks - 1) / ks > cap_blocks) ks *= 2;
  if ((p.bpr + ks - 1) / ks > cap_blocks) return 1;  // row too long for this kernel: caller falls back
  p.ks = ks;
  p.ks_shift = ks == 1 ? 0 : (ks == 2 ? 1 : (ks == 4 ? 2 : 3));
  p.rl = G1_WARPS / ks;
  // balanced split (bpr >= ks always holds: ks > 1 only when bpr exceeds cap_blocks >= 4)
  p.slice_q = p.bpr / ks;
  p.slice_r = p.bpr % ks;
  const int slice_bytes = (p.slice_q + (p.slice_r ? 1 : 0)) * TS;   // the longest slice
  int R = rows_env < 1 ? 1 : (rows_env > G1_R ? G1_R : rows_env);
  // An item is as large as two stages per warp allow with two CTAs on an SM (16 stages in 113 KB less
  // the tables, the staged results and the barriers: 6.9 KB, 3.9 KB with the 48 KB of IQ2_XXS code-book
  // copies).  Larger items mean fewer barrier round trips per warp: 57344x4096 Q4_K 25.1 -> 21.8 us,
  // 14336x4096 8.3 -> 7.8 us with three rows instead of two.
  const size_t tables = TYPE == T_IQ2_XXS ? (size_t)(256 + 128) * 8 * G1_TAB_COPIES : 0;
  p.partial_bytes = (ks > 1 || p.world > 0) ? G1_BATCH * 8 * G1_R * MV * 4 : 0;
  const int room2 = (int)(((size_t)113 * 1024 - tables - (size_t)p.partial_bytes - (size_t)G1_WARPS * 8 * 16) / (2 * G1_WARPS)) - 48;
  const int item_cap = item_env < room2 ? item_env : room2;
  while (R > 1 && (int64_t)R * (ks == 1 ? slice_bytes : (int)round_up(slice_bytes + 32, 16)) > item_cap) --R;
  p.rows_per_item = R;
  p.inv_r = R == 1 ? 0u : (unsigned)(((1ull << 32) + R - 1) / R);
  p.slot_bytes = ks == 1 ? slice_bytes : (int)round_up(slice_bytes + 32, 16);
  p.stage_bytes = ks == 1 ? (int)round_up((int64_t)R * slice_bytes + 32, 16) : R * p.slot_bytes;
  const int kpad = (int)round_up(p.k, 512);
  p.x_bytes = p.x_raw ? (int)round_up((int64_t)MV * (kpad + kpad / 4), 128) : 0;
  p.x_alias = (p.x_raw && p.x_bytes <= p.stage_bytes) ? 1 : 0;
  if (p.x_alias) p.x_bytes = 0;
  const size_t fixed = tables + (size_t)p.x_bytes + (size_t)p.partial_bytes + (size_t)G1_WARPS * 8 * 16;   // + barriers (at most 16 stages)
  auto kern = gemv1_kernel<TYPE, out_t, MV>;
  // Grid first (it decides how many items a warp gets), then the ring depth: as many stages as a
  // warp has items, within what leaves room for two CTAs per SM; GGUF_B200_GEMV1_STAGES caps it.
  const size_t budget2 = (size_t)113 * 1024;
  int per_sm = ctas_env < 1 ? 1 : (ctas_env > 2 ? 2 : ctas_env);
  if (fixed + (size_t)G1_WARPS * 2 * p.stage_bytes > budget2) {
    if (p.x_raw) return 1;   // quantizing in the kernel would cost the second CTA of every SM: the caller quantizes separately
    per_sm = 1;
  }
  int64_t grid = 148 * per_sm;
  const int64_t groups = (p.n + R - 1) / R;
  const int64_t need = (groups + p.rl - 1) / p.rl;
  if (grid > need) grid = need;
  if (grid < 1) grid = 1;
  const int64_t rows_per_lane = (p.n + grid * p.rl - 1) / (grid * p.rl);
  int want = (int)((rows_per_lane + R - 1) / R);
  const int cap = stages_env < 2 ? 16 : (stages_env > 16 ? 16 : stages_env);
  if (want > cap) want = cap;
  if (want < 2) want = 2;
  const size_t room = (per_sm == 2 ? budget2 : (size_t)226 * 1024) - fixed;
  int fit = (int)(room / ((size_t)G1_WARPS * p.stage_bytes));
  if (fit < 2) return 1;   // not even a double buffer: the general kernel takes the shape
  p.stages = want < fit ? want : fit;
  auto smem_of = [&](int stages) { return tables + (size_t)p.x_bytes + (size_t)p.partial_bytes + (size_t)G1_WARPS * stages * p.stage_bytes + (size_t)G1_WARPS * stages * 8; };
  int dev = 0;
  cudaGetDevice(&dev);
  static bool carveout_set[64] = {false};
  if (!carveout_set[dev & 63]) {   // two CTAs of up to 113 KB need (almost) the whole SM as shared memory
    if (cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared) != cudaSuccess) return E_CUDA;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess) return E_CUDA;
    carveout_set[dev & 63] = true;
  }
  // the deeper ring must not cost the second CTA of an SM: ask the runtime, once per size
  static int checked_stages[64][17];   // [device][wanted stages] -> stages that keep per_sm CTAs resident (0 = not asked yet), for the last stage size seen
  static int checked_bytes[64][17];
  if (per_sm == 2 && p.stages > 2) {
    int& memo = checked_stages[dev & 63][p.stages];
    int& memo_b = checked_bytes[dev & 63][p.stages];
    if (memo == 0 || memo_b != p.stage_bytes + p.partial_bytes + p.x_bytes + (int)tables) {
      int st = p.stages, nb = 0;
      while (st > 2) {
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, kern, G1_WARPS * 32, smem_of(st)) != cudaSuccess) return E_CUDA;
        if (nb >= 2) break;
        --st;
      }
      memo = st;
      memo_b = p.stage_bytes + p.partial_bytes + p.x_bytes + (int)tables;
    }
    p.stages = memo;
  }
  const size_t smem = smem_of(p.stages);
  if (smem > 227 * 1024) return 1;
  unsigned gy = 1;
  if (p.topk_ids) {   // MoE decode: the CTAs are shared out over the (token, expert) pairs
    gy = (unsigned)p.moe_slots;
    const int64_t per_pair = (148 * per_sm + gy - 1) / gy;
    if (grid > per_pair) grid = per_pair;
  }
  if (p.n > 0x7fffff00ll) return 1;   // rows are counted in 32 bits
  p.q_rows = (int)(p.n / (grid * p.rl));
  p.r_rows = (int)(p.n % (grid * p.rl));
  return launch_pdl(kern, dim3((unsigned)grid, gy), dim3(G1_WARPS * 32), smem, stream, p) == cudaSuccess ? E_OK : E_CUDA;
}

template <int TYPE>
static int launch_g1_out(const G1Params& p, int out_dtype, int mv, cudaStream_t s) {
  if (mv == 2) {
    switch (out_dtype) {
      case DT_F32: return launch_g1<TYPE, float, 2>(p, s);
      case DT_F16: return launch_g1<TYPE, __half, 2>(p, s);
      case DT_BF16: return launch_g1<TYPE, __nv_bfloat16, 2>(p, s);
    }
    return E_BAD_DTYPE;
  }
  switch (out_dtype) {
    case DT_F32: return launch_g1<TYPE, float, 1>(p, s);
    case DT_F16: return launch_g1<TYPE, __half, 1>(p, s);
    case DT_BF16: return launch_g1<TYPE, __nv_bfloat16, 1>(p, s);
  }
  return E_BAD_DTYPE;
}

// Returns E_OK, a negative error, or 1 when the shape is outside this kernel's reach.
int launch_gemv1(const void* w, const void* xq_soa, void* y, int type, int out_dtype, int64_t N, int64_t K, int* status,
                 cudaStream_t stream, const GemvTp* tp, int vectors, const GemvMoe* moe, int vec0, int total_vecs,
                 const void* x_raw, int x_sum_mode) {
  G1Params p{};
  p.x_raw = x_raw;
  p.x_sum_mode = x_sum_mode;
  if (vectors != 1 && (vectors != 2 || tp || moe)) return 1;
  p.xq_vecs = total_vecs > 0 ? total_vecs : vectors;
  p.vec0 = vec0;
  if (moe) {
    if (tp) return 1;
    const int64_t eb = N * (K / block_size(type)) * type_size(type);
    if (eb % 16 != 0 || moe->slots > 65535) return 1;   // experts must start on 16-byte boundaries; grid.y limit
    p.topk_ids = moe->topk_ids;
    p.top_k = (int)moe->top_k;
    p.n_experts = (int)moe->n_experts;
    p.xq_vecs = (int)moe->tokens;
    p.moe_slots = (int)moe->slots;
    p.expert_bytes = eb;
  }
  if (tp) {
    if (tp->world < 1 || tp->world > G1_MAX_WORLD || tp->slot < 0) return E_BAD_SHAPE;
    p.world = tp->world;
    p.slot = tp->slot;
    p.epoch = tp->epoch;
    p.y_off = tp->y_off;
    for (int r = 0; r < tp->world; ++r) p.ll_peer[r] = tp->ll_peer[r];
  }
  p.w = static_cast<const uint8_t*>(w);
  p.bpr = (int)(K / block_size(type));
  p.w_bytes = N * p.bpr * type_size(type);
  p.xq = static_cast<const uint8_t*>(xq_soa);
  p.y = y;
  p.n = N;
  p.k = K;
  p.status = status;
  switch (type) {
    case T_Q4_0: return launch_g1_out<T_Q4_0>(p, out_dtype, vectors, stream);
    case T_Q8_0: return launch_g1_out<T_Q8_0>(p, out_dtype, vectors, stream);
    case T_Q4_K: return launch_g1_out<T_Q4_K>(p, out_dtype, vectors, stream);
    case T_Q6_K: return launch_g1_out<T_Q6_K>(p, out_dtype, vectors, stream);
    case T_IQ2_XXS: return launch_g1_out<T_IQ2_XXS>(p, out_dtype, vectors, stream);
    case T_IQ4_XS: return launch_g1_out<T_IQ4_XS>(p, out_dtype, vectors, stream);
    case T_Q4_1: return launch_g1_out<T_Q4_1>(p, out_dtype, vectors, stream);
    case T_Q5_0: return launch_g1_out<T_Q5_0>(p, out_dtype, vectors, stream);
    case T_Q5_1: return launch_g1_out<T_Q5_1>(p, out_dtype, vectors, stream);
    case T_Q5_K: return launch_g1_out<T_Q5_K>(p, out_dtype, vectors, stream);
    case T_IQ4_NL: return launch_g1_out<T_IQ4_NL>(p, out_dtype, vectors, stream);
    case T_Q2_K: return launch_g1_out<T_Q2_K>(p, out_dtype, vectors, stream);
    case T_Q3_K: return launch_g1_out<T_Q3_K>(p, out_dtype, vectors, stream);
    case T_IQ2_XS: return launch_g1_out<T_IQ2_XS>(p, out_dtype, vectors, stream);
    case T_IQ2_S: return launch_g1_out<T_IQ2_S>(p, out_dtype, vectors, stream);
    case T_IQ3_XXS: return launch_g1_out<T_IQ3_XXS>(p, out_dtype, vectors, stream);
    case T_IQ3_S: return launch_g1_out<T_IQ3_S>(p, out_dtype, vectors, stream);
    case T_IQ1_S: return launch_g1_out<T_IQ1_S>(p, out_dtype, vectors, stream);
    case T_IQ1_M: return launch_g1_out<T_IQ1_M>(p, out_dtype, vectors, stream);
  }
  return E_BAD_TYPE;
}

}  // namespace gguf_b200
