/*
 * CPU oracle for the GGUF quantized-matmul hot path.  TEST INFRASTRUCTURE ONLY:
 * nothing in the product library links, loads or calls this file; it exists so that
 * tests (and the CPU-baseline leg of the benchmark) can check the CUDA kernels.
 *
 * It restates, in plain C, the arithmetic of the reference plugin's CUDA kernels
 * (vllm_gguf_plugin/csrc/gguf/ of akmorley/vllm-gguf-plugin-prism) for these block types:
 *   Q4_0 (2), Q8_0 (8), Q4_K (12), Q6_K (14), IQ2_XXS (16), IQ4_XS (23), and later additions
 *   (Q4_1, Q5_0, Q5_1, Q2_K, Q3_K, Q5_K, IQ4_NL, IQ2_XS, IQ2_S, IQ3_XXS, IQ3_S, IQ1_S, IQ1_M).
 * Each function names the reference lines it follows.  Half-precision steps are
 * emulated exactly (one IEEE rounding per __hmul/__hsub/__int2half_rn), so the
 * dequantize outputs are bit patterns, not approximations.  Matmul entry points are
 * evaluated in double precision: they give the value the reference formulas define,
 * free of the fp32 summation-order noise of any particular GPU schedule.
 *
 * Pinning: the reference holds no self-contained golden vectors for this path (its
 * kernel tests need fixture files from a model hub).  The oracle is pinned instead
 *  (1) against gguf-py's dequantize (the third-party format definition the reference's
 *      own tests compare with, tests/test_kernels.py:77-99) on committed fixtures, and
 *  (2) on a GPU, against the reference's own kernels built by oracle/build_ref.py.
 *
 * Known, documented gap: the reference is compiled with --use_fast_math, so the two
 * fp32 divisions of its q8_1 quantizer are approximate on the GPU; this file uses
 * IEEE division.  Differences are confined to near-ties and are classified by the
 * tests (the GPU-vs-reference-GPU comparison is bit-exact).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "../include/gguf_b200_iq_tables.h"

#define QK 32
#define QK_K 256

enum { T_Q4_0 = 2, T_Q4_1 = 3, T_Q5_0 = 6, T_Q5_1 = 7, T_Q8_0 = 8, T_Q2_K = 10, T_Q3_K = 11, T_Q4_K = 12, T_Q5_K = 13, T_Q6_K = 14,
       T_IQ2_XXS = 16, T_IQ2_XS = 17, T_IQ3_XXS = 18, T_IQ1_S = 19, T_IQ4_NL = 20, T_IQ3_S = 21, T_IQ2_S = 22, T_IQ4_XS = 23,
       T_IQ1_M = 29 };
enum { DT_F32 = 0, DT_F16 = 1, DT_BF16 = 2 };

/* ------------------------------------------------------------------ */
/* exact half / bfloat16 helpers                                       */
/* ------------------------------------------------------------------ */

typedef __int128 i128;
typedef unsigned __int128 u128;

static float h2f(uint16_t h) {
  uint32_t s = (uint32_t)(h >> 15) << 31, e = (h >> 10) & 31, m = h & 1023, u;
  if (e == 0) {
    if (m == 0) {
      u = s;
    } else { /* subnormal: value = m * 2^-24 */
      float f = (float)m * 5.9604644775390625e-08f;
      memcpy(&u, &f, 4);
      u |= s;
    }
  } else if (e == 31) {
    u = s | 0x7f800000u | (m << 13);
  } else {
    u = s | ((e + 112) << 23) | (m << 13);
  }
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* A finite half as an integer in units of 2^-48 (so that products of two halves,
 * whose smallest bit is 2^-48, are integers too). */
static i128 h2s(uint16_t h) {
  int e = (h >> 10) & 31, m = h & 1023;
  i128 v = (e == 0) ? ((i128)m << 24) : ((i128)(m | 1024) << (e - 1 + 24));
  return (h & 0x8000) ? -v : v;
}

/* Round an exact value (units of 2^-48) to half, round-to-nearest-even. */
static uint16_t s2h(i128 v) {
  uint16_t sign = 0;
  if (v < 0) {
    sign = 0x8000;
    v = -v;
  }
  u128 m = (u128)v;
  if (m == 0) return sign;
  int p = 127;
  while (!((m >> p) & 1)) --p; /* msb position */
  int e = p - 48;             /* value in [2^e, 2^(e+1)) */
  int shift = (e < -14) ? 24 : (p - 10);
  u128 q = m >> shift, rem = m & (((u128)1 << shift) - 1), half = (u128)1 << (shift - 1);
  if (shift == 0) {
    rem = 0;
    half = 1;
  }
  if (rem > half || (rem == half && (q & 1))) ++q;
  if (e < -14) return sign | (uint16_t)q; /* subnormal (q==1024 carries into the first normal) */
  if (q == 2048) {
    q = 1024;
    ++e;
  }
  if (e > 15) return sign | 0x7c00;
  return sign | (uint16_t)(((e + 15) << 10) | ((int)q & 1023));
}

/* IEEE sign of an exact zero: a product keeps the xor of the signs; a sum of two zeros of
 * equal sign keeps it, any other exact cancellation gives +0 (round-to-nearest). */
static uint16_t hmul(uint16_t a, uint16_t b) { /* one rounding, like mul.f16 */
  i128 pa = h2s(a) >> 24, pb = h2s(b) >> 24;   /* back to units of 2^-24 each */
  i128 p = pa * pb;
  if (p == 0) return (uint16_t)((a ^ b) & 0x8000);
  return s2h(p);
}
static uint16_t hsub(uint16_t a, uint16_t b) {
  i128 v = h2s(a) - h2s(b);
  if (v == 0) return (uint16_t)(((a & 0x8000) && !(b & 0x8000)) ? 0x8000 : 0); /* (-0) - (+0) = -0 */
  return s2h(v);
}
static uint16_t hfms(uint16_t a, uint16_t b, uint16_t c) { /* a*b - c with a single rounding */
  i128 pa = h2s(a) >> 24, pb = h2s(b) >> 24;
  i128 v = pa * pb - h2s(c);
  if (v == 0) {
    const int sp = ((a ^ b) & 0x8000) != 0, sc = !(c & 0x8000); /* signs of the product and of -c */
    const int both_zero = (pa * pb == 0);
    return (uint16_t)((both_zero && sp && sc) ? 0x8000 : 0);
  }
  return s2h(v);
}
static uint16_t i2h(int v) { return s2h((i128)v << 48); } /* __int2half_rn */
static uint16_t hneg(uint16_t a) { return (uint16_t)(a ^ 0x8000); }
static uint16_t hadd(uint16_t a, uint16_t b) { return hsub(a, hneg(b)); }
static uint16_t hfma(uint16_t a, uint16_t b, uint16_t c) { return hfms(a, b, hneg(c)); } /* a*b + c, one rounding */

static uint16_t f2h(float f) { /* __float2half_rn */
  uint32_t u;
  memcpy(&u, &f, 4);
  uint16_t sign = (uint16_t)((u >> 16) & 0x8000);
  uint32_t e = (u >> 23) & 255, m = u & 0x7fffff;
  if (e == 255) return sign | 0x7c00 | (m ? 0x200 : 0);
  if (e == 0) return sign; /* fp32 subnormals are below half the smallest half subnormal */
  int E = (int)e - 127;
  if (E > 15) return sign | 0x7c00;
  if (E < -25) return sign;
  /* finite, within reach: 24-bit significand M * 2^(E-23); bring to units of 2^-48 */
  u128 M = (u128)(m | 0x800000);
  int sh = E - 23 + 48; /* >= 0 because E >= -25 */
  uint16_t r = s2h((i128)(M << sh));
  return sign | r;
}

static uint16_t f2bf(float f) { /* __float2bfloat16_rn */
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffff) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
  u += 0x7fff + ((u >> 16) & 1);
  return (uint16_t)(u >> 16);
}
static float bf2f(uint16_t b) {
  uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

static float load_act(const void* x, int dt, int64_t i) {
  if (dt == DT_F32) return ((const float*)x)[i];
  if (dt == DT_F16) return h2f(((const uint16_t*)x)[i]);
  return bf2f(((const uint16_t*)x)[i]);
}

/* store a value that is already a half (half-arithmetic decoders):
 * convert_from_half<dst_t>, ggml-common.h:1079-1096 */
static void store_h(void* out, int dt, int64_t i, uint16_t h) {
  if (dt == DT_F16)
    ((uint16_t*)out)[i] = h;
  else if (dt == DT_F32)
    ((float*)out)[i] = h2f(h);
  else
    ((uint16_t*)out)[i] = f2bf(h2f(h));
}
/* store an fp32 value by implicit conversion to dst_t (fp32-arithmetic decoders and all
 * matmul outputs, e.g. mmvq.cuh:38-40) */
static void store_f(void* out, int dt, int64_t i, float f) {
  if (dt == DT_F32)
    ((float*)out)[i] = f;
  else if (dt == DT_F16)
    ((uint16_t*)out)[i] = f2h(f);
  else
    ((uint16_t*)out)[i] = f2bf(f);
}

static uint16_t rd16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }

int oracle_type_size(int type) {
  switch (type) {
    case T_Q4_0: return 18;
    case T_Q8_0: return 34;
    case T_Q4_K: return 144;
    case T_Q6_K: return 210;
    case T_IQ2_XXS: return 66;
    case T_IQ4_XS: return 136;
    case T_Q4_1: return 20;
    case T_Q5_0: return 22;
    case T_Q5_1: return 24;
    case T_Q2_K: return 84;
    case T_Q3_K: return 110;
    case T_Q5_K: return 176;
    case T_IQ4_NL: return 18;
    case T_IQ2_XS: return 74;
    case T_IQ2_S: return 82;
    case T_IQ3_XXS: return 98;
    case T_IQ3_S: return 110;
    case T_IQ1_S: return 50;
    case T_IQ1_M: return 56;
  }
  return 0;
}
int oracle_block_size(int type) {
  switch (type) {
    case T_Q4_0: case T_Q4_1: case T_Q5_0: case T_Q5_1: case T_Q8_0: case T_IQ4_NL: return QK;
  }
  return oracle_type_size(type) ? QK_K : 0;
}

/* 6-bit (scale, min) pair j of a Q4_K super-block: get_scale_min_k4, dequantize.cuh:156-163 */
static void scale_min_k4(int j, const uint8_t* q, int* sc, int* m) {
  if (j < 4) {
    *sc = q[j] & 63;
    *m = q[j + 4] & 63;
  } else {
    *sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4);
    *m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
  }
}

/* 6-bit sub-block scale of IQ4_XS minus 32: dequantize.cuh:429, vecdotq.cuh:1801 */
static int iq4xs_ls(const uint8_t* blk, int ib) {
  uint16_t sh = rd16(blk + 2);
  const uint8_t* sl = blk + 4;
  return (((sl[ib / 2] >> (4 * (ib % 2))) & 0xf) | (((sh >> (2 * ib)) & 3) << 4)) - 32;
}

/* ------------------------------------------------------------------ */
/* standalone dequantize (ggml_dequantize, gguf_kernel.cu:87-102)      */
/* ------------------------------------------------------------------ */

/* q4k_contract: 0 = __hmul then __hsub with two roundings (dequantize.cuh:193-194 as
 * written); 1 = the same pair contracted into one fused multiply-subtract, which the PTX
 * rules allow the assembler to do for mul.f16/sub.f16 without an explicit .rn.  Which of
 * the two the reference binary does is decided on the GPU by comparing with it: on sm_100a
 * (nvcc 12.9, reference flags) it is 1, the fused form. */
int oracle_dequantize(const uint8_t* w, int type, void* out, int out_dt, int64_t n_elems,
                      int q4k_contract) {
  const int ts = oracle_type_size(type), bs = oracle_block_size(type);
  if (!ts) return -1;
  const int64_t nb = n_elems / bs;
  for (int64_t b = 0; b < nb; ++b) {
    const uint8_t* blk = w + b * ts;
    const int64_t o = b * bs;
    switch (type) {
      case T_Q4_0: { /* dequantize_q4_0, dequantize.cuh:3-15; placement :88-98 */
        uint16_t d = rd16(blk);
        for (int j = 0; j < 16; ++j) {
          int q = blk[2 + j];
          store_h(out, out_dt, o + j, hmul(hsub(i2h(q & 0xF), i2h(8)), d));
          store_h(out, out_dt, o + j + 16, hmul(hsub(i2h(q >> 4), i2h(8)), d));
        }
      } break;
      case T_Q8_0: { /* dequantize_q8_0, dequantize.cuh:69-78 */
        uint16_t d = rd16(blk);
        for (int j = 0; j < 32; ++j) store_h(out, out_dt, o + j, hmul(i2h((int8_t)blk[2 + j]), d));
      } break;
      case T_Q4_K: { /* dequantize_block_q4_K, dequantize.cuh:165-196 */
        uint16_t dall = rd16(blk), dmin = rd16(blk + 2);
        const uint8_t *scales = blk + 4, *qs = blk + 16;
        for (int il = 0; il < 4; ++il) {
          int sc, m;
          scale_min_k4(2 * il, scales, &sc, &m);
          uint16_t d1 = hmul(dall, i2h(sc)), m1 = hmul(dmin, i2h(m));
          scale_min_k4(2 * il + 1, scales, &sc, &m);
          uint16_t d2 = hmul(dall, i2h(sc)), m2 = hmul(dmin, i2h(m));
          for (int l = 0; l < 32; ++l) {
            int q = qs[32 * il + l];
            uint16_t lo, hi;
            if (q4k_contract) {
              lo = hfms(d1, i2h(q & 0xF), m1);
              hi = hfms(d2, i2h(q >> 4), m2);
            } else {
              lo = hsub(hmul(d1, i2h(q & 0xF)), m1);
              hi = hsub(hmul(d2, i2h(q >> 4)), m2);
            }
            store_h(out, out_dt, o + 64 * il + l, lo);
            store_h(out, out_dt, o + 64 * il + 32 + l, hi);
          }
        }
      } break;
      case T_Q6_K: { /* dequantize_block_q6_K, dequantize.cuh:232-256 */
        const uint8_t *ql = blk, *qh = blk + 128;
        const int8_t* sc = (const int8_t*)(blk + 192);
        uint16_t d = rd16(blk + 208);
        for (int ip = 0; ip < 2; ++ip)
          for (int il = 0; il < 32; ++il) {
            int is = 8 * ip + il / 16;
            int l0 = ql[64 * ip + il], l1 = ql[64 * ip + il + 32], h = qh[32 * ip + il];
            int q0 = (int8_t)((l0 & 0xF) | (((h >> 0) & 3) << 4)) - 32;
            int q1 = (int8_t)((l1 & 0xF) | (((h >> 2) & 3) << 4)) - 32;
            int q2 = (int8_t)((l0 >> 4) | (((h >> 4) & 3) << 4)) - 32;
            int q3 = (int8_t)((l1 >> 4) | (((h >> 6) & 3) << 4)) - 32;
            int64_t y = o + 128 * ip + il;
            store_h(out, out_dt, y + 0, hmul(d, i2h(sc[is + 0] * q0)));
            store_h(out, out_dt, y + 32, hmul(d, i2h(sc[is + 2] * q1)));
            store_h(out, out_dt, y + 64, hmul(d, i2h(sc[is + 4] * q2)));
            store_h(out, out_dt, y + 96, hmul(d, i2h(sc[is + 6] * q3)));
          }
      } break;
      case T_IQ2_XXS: { /* dequantize_block_iq2_xxs, dequantize.cuh:258-275 (fp32 math) */
        float df = h2f(rd16(blk));
        for (int ib = 0; ib < 8; ++ib) {
          const uint8_t* q2 = blk + 2 + 8 * ib;
          uint32_t aux32 = (uint32_t)q2[4] | ((uint32_t)q2[5] << 8) | ((uint32_t)q2[6] << 16) | ((uint32_t)q2[7] << 24);
          volatile float d = df * (0.5f + (float)(aux32 >> 28));
          d = d * 0.25f;
          for (int il = 0; il < 4; ++il) {
            uint64_t grid = gguf_b200_iq2xxs_grid[q2[il]];
            uint8_t signs = gguf_b200_ksigns_iq2xs[(aux32 >> (7 * il)) & 127];
            for (int j = 0; j < 8; ++j) {
              volatile float v = d * (float)((grid >> (8 * j)) & 0xff);
              v = v * ((signs >> j) & 1 ? -1.f : 1.f);
              store_f(out, out_dt, o + 32 * ib + 8 * il + j, v);
            }
          }
        }
      } break;
      case T_IQ2_XS: case T_IQ2_S: case T_IQ3_XXS: case T_IQ3_S: {
        /* dequantize_block_iq2_xs / iq2_s / iq3_xxs / iq3_s, dequantize.cuh:277-353: per group of 8
         * values (ib = sub-block of 32, il = group) y[j] = d * grid[j] * sign(j) in fp32, with
         * d = half2float(x.d) * (0.5f + scale) * 0.25f (IQ2) or * 0.5f (IQ3). */
        float df = h2f(rd16(blk));
        for (int ib = 0; ib < 8; ++ib)
          for (int il = 0; il < 4; ++il) {
            uint64_t grid;
            uint32_t signs, sc;
            float mul;
            if (type == T_IQ2_XS) {          /* half d | u16 qs[32] | u8 scales[8] */
              uint32_t q = rd16(blk + 2 + 2 * (4 * ib + il));
              grid = gguf_b200_iq2xs_grid[q & 511];
              signs = gguf_b200_ksigns_iq2xs[q >> 9];
              sc = (blk[66 + ib] >> (4 * (il / 2))) & 0xf;
              mul = 0.25f;
            } else if (type == T_IQ2_S) {    /* half d | u8 qs[64] (32 indices, 32 sign bytes) | u8 qh[8] | u8 scales[8] */
              grid = gguf_b200_iq2s_grid[blk[2 + 4 * ib + il] | (((uint32_t)blk[66 + ib] << (8 - 2 * il)) & 0x300)];
              signs = blk[2 + 32 + 4 * ib + il];
              sc = (blk[74 + ib] >> (4 * (il / 2))) & 0xf;
              mul = 0.25f;
            } else if (type == T_IQ3_XXS) {  /* half d | u8 qs[64] | u32 scale+signs [8] */
              const uint8_t* q3 = blk + 2 + 8 * ib;
              const uint8_t* g = blk + 2 + 64 + 4 * ib;
              uint32_t aux32 = (uint32_t)g[0] | ((uint32_t)g[1] << 8) | ((uint32_t)g[2] << 16) | ((uint32_t)g[3] << 24);
              grid = (uint64_t)gguf_b200_iq3xxs_grid[q3[2 * il]] | ((uint64_t)gguf_b200_iq3xxs_grid[q3[2 * il + 1]] << 32);
              signs = gguf_b200_ksigns_iq2xs[(aux32 >> (7 * il)) & 127];
              sc = aux32 >> 28;
              mul = 0.5f;
            } else {                         /* half d | u8 qs[64] | u8 qh[8] | u8 signs[32] | u8 scales[4] */
              const uint8_t* qs = blk + 2 + 8 * ib;
              uint32_t qh = blk[66 + ib];
              grid = (uint64_t)gguf_b200_iq3s_grid[qs[2 * il] | ((qh << (8 - 2 * il)) & 256)] |
                     ((uint64_t)gguf_b200_iq3s_grid[qs[2 * il + 1] | ((qh << (7 - 2 * il)) & 256)] << 32);
              signs = blk[74 + 4 * ib + il];
              sc = (blk[106 + ib / 2] >> (4 * (ib % 2))) & 0xf;
              mul = 0.5f;
            }
            volatile float d = df * (0.5f + (float)sc);
            d = d * mul;
            for (int j = 0; j < 8; ++j) {
              volatile float v = d * (float)((grid >> (8 * j)) & 0xff);
              v = v * ((signs >> j) & 1 ? -1.f : 1.f);
              store_f(out, out_dt, o + 32 * ib + 8 * il + j, v);
            }
          }
      } break;
      case T_IQ1_S: case T_IQ1_M: {
        /* dequantize_block_iq1_s / iq1_m, dequantize.cuh:355-399: y[j] = d * (q[j] + delta), q in {0,1,2}
         * nibble-packed in the code book, delta = -1 - 1/8 or -1 + 1/8, d = scale * (2 * s3 + 1). */
        for (int ib = 0; ib < 8; ++ib)
          for (int il = 0; il < 4; ++il) {
            volatile float d;
            float delta;
            uint32_t g;
            if (type == T_IQ1_S) {           /* half d | u8 qs[32] | u16 qh[8] */
              uint32_t qh = rd16(blk + 34 + 2 * ib);
              delta = (qh & 0x8000) ? -1.f - 0.125f : -1.f + 0.125f;
              d = h2f(rd16(blk)) * (float)(2 * ((qh >> 12) & 7) + 1);
              g = gguf_b200_iq1s_grid[blk[2 + 4 * ib + il] | (((qh >> (3 * il)) & 7) << 8)];
            } else {                         /* u8 qs[32] | u8 qh[16] | u16 scales[4] */
              uint32_t sc0 = rd16(blk + 48), sc1 = rd16(blk + 50), sc2 = rd16(blk + 52), sc3 = rd16(blk + 54);
              uint16_t s16 = (uint16_t)((sc0 >> 12) | ((sc1 >> 8) & 0x00f0) | ((sc2 >> 4) & 0x0f00) | (sc3 & 0xf000));
              int ib16 = 2 * ib + il / 2;
              uint32_t scw = rd16(blk + 48 + 2 * (ib16 / 4));
              d = h2f(s16) * (float)(2 * ((scw >> (3 * (ib16 % 4))) & 7) + 1);
              uint32_t qh = blk[32 + 2 * ib + il / 2];
              delta = (qh & (0x08u << (4 * (il % 2)))) ? -1.f - 0.125f : -1.f + 0.125f;
              g = gguf_b200_iq1s_grid[blk[4 * ib + il] | (((qh >> (4 * (il % 2))) & 7) << 8)];
            }
            for (int j = 0; j < 8; ++j) {
              volatile float q = (float)((g >> (8 * (j & 3) + 4 * (j >> 2))) & 0xf) + delta;
              volatile float v = d * q;
              store_f(out, out_dt, o + 32 * ib + 8 * il + j, v);
            }
          }
      } break;
      case T_Q4_1: { /* dequantize_q4_1, dequantize.cuh:17-31: v = q*d + m (contract: one fused multiply-add) */
        uint16_t d = rd16(blk), m = rd16(blk + 2);
        for (int j = 0; j < 16; ++j) {
          int q = blk[4 + j];
          store_h(out, out_dt, o + j, q4k_contract ? hfma(i2h(q & 0xF), d, m) : hadd(hmul(i2h(q & 0xF), d), m));
          store_h(out, out_dt, o + j + 16, q4k_contract ? hfma(i2h(q >> 4), d, m) : hadd(hmul(i2h(q >> 4), d), m));
        }
      } break;
      case T_Q5_0:   /* dequantize_q5_0, dequantize.cuh:33-50: (q - 16) * d */
      case T_Q5_1: { /* dequantize_q5_1, dequantize.cuh:52-69: q * d + m */
        const int one = type == T_Q5_1;
        uint16_t d = rd16(blk), m = one ? rd16(blk + 2) : 0;
        const uint8_t* qhp = blk + (one ? 4 : 2);
        const uint8_t* qs = blk + (one ? 8 : 6);
        uint32_t qh = (uint32_t)qhp[0] | ((uint32_t)qhp[1] << 8) | ((uint32_t)qhp[2] << 16) | ((uint32_t)qhp[3] << 24);
        for (int j = 0; j < 16; ++j) {
          int x0 = (qs[j] & 0xF) | (((qh >> j) << 4) & 0x10);
          int x1 = (qs[j] >> 4) | ((qh >> (j + 12)) & 0x10);
          uint16_t v0, v1;
          if (one) {
            v0 = q4k_contract ? hfma(i2h(x0), d, m) : hadd(hmul(i2h(x0), d), m);
            v1 = q4k_contract ? hfma(i2h(x1), d, m) : hadd(hmul(i2h(x1), d), m);
          } else {
            v0 = hmul(hsub(i2h(x0), i2h(16)), d);
            v1 = hmul(hsub(i2h(x1), i2h(16)), d);
          }
          store_h(out, out_dt, o + j, v0);
          store_h(out, out_dt, o + j + 16, v1);
        }
      } break;
      case T_Q2_K: { /* dequantize_block_q2_K, dequantize.cuh:101-120: dall*(sc&15)*q - dmin*(sc>>4) */
        const uint8_t *scales = blk, *qs = blk + 16;
        uint16_t dall = rd16(blk + 80), dmin = rd16(blk + 82);
        for (int n = 0; n < 2; ++n)
          for (int l = 0; l < 32; ++l) {
            int is = 8 * n + l / 16;
            int q = qs[32 * n + l];
            for (int k = 0; k < 4; ++k) {
              int sc = scales[is + 2 * k];
              uint16_t a = i2h((sc & 0xF) * ((q >> (2 * k)) & 3)), mm = hmul(dmin, i2h(sc >> 4));
              /* contraction: the subtraction fuses with the FIRST product (a*dall - mm in one rounding) */
              uint16_t v = q4k_contract ? hfms(dall, a, mm) : hsub(hmul(dall, a), mm);
              store_h(out, out_dt, o + 128 * n + l + 32 * k, v);
            }
          }
      } break;
      case T_Q3_K: { /* dequantize_block_q3_K, dequantize.cuh:122-154 */
        const uint8_t *hm = blk, *qs = blk + 32, *sc = blk + 96;
        uint16_t d_all = rd16(blk + 108);
        for (int n = 0; n < 2; ++n)
          for (int j = 0; j < 4; ++j)
            for (int is0 = 0; is0 < 2; ++is0) {
              int is = 8 * n + 2 * j + is0, us;
              if (is < 4) us = (sc[is] & 0xF) | (((sc[is + 8] >> 0) & 3) << 4);
              else if (is < 8) us = (sc[is] & 0xF) | (((sc[is + 4] >> 2) & 3) << 4);
              else if (is < 12) us = (sc[is - 8] >> 4) | (((sc[is] >> 4) & 3) << 4);
              else us = (sc[is - 8] >> 4) | (((sc[is - 4] >> 6) & 3) << 4);
              uint16_t dl = hmul(d_all, i2h((int8_t)us - 32));
              int m = 1 << (4 * n + j);
              for (int l = 16 * is0; l < 16 * is0 + 16; ++l) {
                int v = (int8_t)((qs[32 * n + l] >> (2 * j)) & 3) - ((hm[l] & m) ? 0 : 4);
                store_h(out, out_dt, o + 128 * n + 32 * j + l, hmul(dl, i2h(v)));
              }
            }
      } break;
      case T_Q5_K: { /* dequantize_block_q5_K, dequantize.cuh:198-230 */
        uint16_t dall = rd16(blk), dmin = rd16(blk + 2);
        const uint8_t *scales = blk + 4, *qh = blk + 16, *qs = blk + 48;
        for (int il = 0; il < 4; ++il) {
          int sc, m;
          scale_min_k4(2 * il, scales, &sc, &m);
          uint16_t d1 = hmul(dall, i2h(sc)), m1 = hmul(dmin, i2h(m));
          scale_min_k4(2 * il + 1, scales, &sc, &m);
          uint16_t d2 = hmul(dall, i2h(sc)), m2 = hmul(dmin, i2h(m));
          for (int l = 0; l < 32; ++l) {
            int lo = (qs[32 * il + l] & 0xF) + ((qh[l] & (1 << (2 * il))) ? 16 : 0);
            int hi = (qs[32 * il + l] >> 4) + ((qh[l] & (2 << (2 * il))) ? 16 : 0);
            store_h(out, out_dt, o + 64 * il + l, q4k_contract ? hfms(d1, i2h(lo), m1) : hsub(hmul(d1, i2h(lo)), m1));
            store_h(out, out_dt, o + 64 * il + 32 + l, q4k_contract ? hfms(d2, i2h(hi), m2) : hsub(hmul(d2, i2h(hi)), m2));
          }
        }
      } break;
      case T_IQ4_NL: { /* dequantize_block_iq4_nl, dequantize.cuh:400-418 (fp32 math) */
        float df = h2f(rd16(blk));
        for (int j = 0; j < 16; ++j) {
          int q = blk[2 + j];
          volatile float lo = df * (float)gguf_b200_kvalues_iq4nl[q & 0xf];
          volatile float hi = df * (float)gguf_b200_kvalues_iq4nl[q >> 4];
          store_f(out, out_dt, o + j, lo);
          store_f(out, out_dt, o + j + 16, hi);
        }
      } break;
      case T_IQ4_XS: { /* dequantize_block_iq4_xs, dequantize.cuh:420-435 (fp32 math) */
        float df = h2f(rd16(blk));
        const uint8_t* qs = blk + 8;
        for (int ib = 0; ib < 8; ++ib) {
          volatile float d = df * (float)iq4xs_ls(blk, ib);
          for (int j = 0; j < 16; ++j) {
            int q = qs[16 * ib + j];
            volatile float lo = d * (float)gguf_b200_kvalues_iq4nl[q & 0xf];
            volatile float hi = d * (float)gguf_b200_kvalues_iq4nl[q >> 4];
            store_f(out, out_dt, o + 32 * ib + j, lo);
            store_f(out, out_dt, o + 32 * ib + j + 16, hi);
          }
        }
      } break;
    }
  }
  return 0;
}

/* ------------------------------------------------------------------ */
/* q8_1 activation quantizer (quantize_q8_1, gguf_kernel.cu:32-69)     */
/* ------------------------------------------------------------------ */

int64_t oracle_q8_1_row_bytes(int64_t K) { return (K + 511) / 512 * 512 / 32 * 36; }

/* out: M rows of Kpad/32 blocks {half d; half sum; int8 qs[32]}, Kpad = K rounded up to
 * 512 (gguf_kernel.cu:74); elements beyond K are zeros (:48).  amax and sum use the
 * xor-butterfly of :53-56 (the order matters for the fp32 sum). */
int oracle_quantize_q8_1(const void* x, int dt, uint8_t* out, int64_t M, int64_t K) {
  const int64_t kpad = (K + 511) / 512 * 512, nb = kpad / 32;
  for (int64_t r = 0; r < M; ++r)
    for (int64_t b = 0; b < nb; ++b) {
      float xi[32], s[32], a[32];
      for (int j = 0; j < 32; ++j) {
        int64_t k = b * 32 + j;
        xi[j] = k < K ? load_act(x, dt, r * K + k) : 0.0f;
        s[j] = xi[j];
        a[j] = fabsf(xi[j]);
      }
      for (int mask = 16; mask > 0; mask >>= 1) {
        float s2[32], a2[32];
        for (int j = 0; j < 32; ++j) {
          volatile float t = s[j] + s[j ^ mask];
          s2[j] = t;
          a2[j] = fmaxf(a[j], a[j ^ mask]);
        }
        memcpy(s, s2, sizeof s);
        memcpy(a, a2, sizeof a);
      }
      const float amax = a[0];
      volatile float d = amax / 127;
      uint8_t* blk = out + (r * nb + b) * 36;
      uint16_t hd = f2h(d), hs = f2h(s[0]);
      blk[0] = hd & 255;
      blk[1] = hd >> 8;
      blk[2] = hs & 255;
      blk[3] = hs >> 8;
      for (int j = 0; j < 32; ++j) {
        volatile float t = xi[j] / d;
        blk[4 + j] = (uint8_t)(int8_t)(amax == 0.0f ? 0 : roundf(t));
      }
    }
  return 0;
}

/* ------------------------------------------------------------------ */
/* block dot products                                                  */
/* ------------------------------------------------------------------ */

static int idot(const int8_t* a, const int8_t* b, int n) {
  int s = 0;
  for (int i = 0; i < n; ++i) s += a[i] * b[i];
  return s;
}

/* Unpack one weight block of `type` to its integer codes w[0..bs) in dequantized order. */
static void unpack_codes(const uint8_t* blk, int type, int8_t* w) {
  switch (type) {
    case T_Q4_0:
      for (int j = 0; j < 16; ++j) {
        w[j] = blk[2 + j] & 0xF;
        w[j + 16] = blk[2 + j] >> 4;
      }
      break;
    case T_Q8_0:
      for (int j = 0; j < 32; ++j) w[j] = (int8_t)blk[2 + j];
      break;
    case T_Q4_K:
      for (int il = 0; il < 4; ++il)
        for (int l = 0; l < 32; ++l) {
          w[64 * il + l] = blk[16 + 32 * il + l] & 0xF;
          w[64 * il + 32 + l] = blk[16 + 32 * il + l] >> 4;
        }
      break;
    case T_Q6_K:
      for (int ip = 0; ip < 2; ++ip)
        for (int il = 0; il < 32; ++il) {
          int l0 = blk[64 * ip + il], l1 = blk[64 * ip + il + 32], h = blk[128 + 32 * ip + il];
          w[128 * ip + il + 0] = (int8_t)(((l0 & 0xF) | (((h >> 0) & 3) << 4)) - 32);
          w[128 * ip + il + 32] = (int8_t)(((l1 & 0xF) | (((h >> 2) & 3) << 4)) - 32);
          w[128 * ip + il + 64] = (int8_t)(((l0 >> 4) | (((h >> 4) & 3) << 4)) - 32);
          w[128 * ip + il + 96] = (int8_t)(((l1 >> 4) | (((h >> 6) & 3) << 4)) - 32);
        }
      break;
    case T_IQ2_XXS:
      for (int ib = 0; ib < 8; ++ib) {
        const uint8_t* q2 = blk + 2 + 8 * ib;
        uint32_t aux32 = (uint32_t)q2[4] | ((uint32_t)q2[5] << 8) | ((uint32_t)q2[6] << 16) | ((uint32_t)q2[7] << 24);
        for (int il = 0; il < 4; ++il) {
          uint64_t grid = gguf_b200_iq2xxs_grid[q2[il]];
          uint8_t signs = gguf_b200_ksigns_iq2xs[(aux32 >> (7 * il)) & 127];
          for (int j = 0; j < 8; ++j) {
            int g = (int)((grid >> (8 * j)) & 0xff);
            w[32 * ib + 8 * il + j] = (int8_t)(((signs >> j) & 1) ? -g : g);
          }
        }
      }
      break;
    case T_IQ4_XS:
      for (int ib = 0; ib < 8; ++ib)
        for (int j = 0; j < 16; ++j) {
          int q = blk[8 + 16 * ib + j];
          w[32 * ib + j] = gguf_b200_kvalues_iq4nl[q & 0xf];
          w[32 * ib + j + 16] = gguf_b200_kvalues_iq4nl[q >> 4];
        }
      break;
    case T_Q4_1:
      for (int j = 0; j < 16; ++j) {
        w[j] = blk[4 + j] & 0xF;
        w[j + 16] = blk[4 + j] >> 4;
      }
      break;
    case T_Q5_0:
    case T_Q5_1: { /* 4 low bits from qs, fifth bit j of qh for value j (vecdotq.cuh:108-122) */
      const uint8_t* qhp = blk + (type == T_Q5_1 ? 4 : 2);
      const uint8_t* qs = blk + (type == T_Q5_1 ? 8 : 6);
      uint32_t qh = (uint32_t)qhp[0] | ((uint32_t)qhp[1] << 8) | ((uint32_t)qhp[2] << 16) | ((uint32_t)qhp[3] << 24);
      for (int j = 0; j < 16; ++j) {
        w[j] = (int8_t)((qs[j] & 0xF) | (((qh >> j) & 1) << 4));
        w[j + 16] = (int8_t)((qs[j] >> 4) | (((qh >> (j + 16)) & 1) << 4));
      }
    } break;
    case T_IQ4_NL:
      for (int j = 0; j < 16; ++j) {
        w[j] = gguf_b200_kvalues_iq4nl[blk[2 + j] & 0xf];
        w[j + 16] = gguf_b200_kvalues_iq4nl[blk[2 + j] >> 4];
      }
      break;
    case T_Q5_K:
      for (int il = 0; il < 4; ++il)
        for (int l = 0; l < 32; ++l) {
          w[64 * il + l] = (int8_t)((blk[48 + 32 * il + l] & 0xF) | (((blk[16 + l] >> (2 * il)) & 1) << 4));
          w[64 * il + 32 + l] = (int8_t)((blk[48 + 32 * il + l] >> 4) | (((blk[16 + l] >> (2 * il + 1)) & 1) << 4));
        }
      break;
    case T_Q2_K: /* scales[16] | qs[64] | d | dmin: value 128n + 32i + l = (qs[32n + l] >> 2i) & 3  (dequantize.cuh:97-118) */
      for (int n = 0; n < 2; ++n)
        for (int i = 0; i < 4; ++i)
          for (int l = 0; l < 32; ++l) w[128 * n + 32 * i + l] = (int8_t)((blk[16 + 32 * n + l] >> (2 * i)) & 3);
      break;
    case T_Q3_K: /* hmask[32] | qs[64] | scales[12] | d: two low bits from qs, minus 4 unless the hmask bit is set
                    (vecdotq.cuh:1024-1048, :269-300) */
      for (int n = 0; n < 2; ++n)
        for (int i = 0; i < 4; ++i)
          for (int l = 0; l < 32; ++l) {
            int q2 = (blk[32 + 32 * n + l] >> (2 * i)) & 3;
            int h = (blk[l] >> (4 * n + i)) & 1;
            w[128 * n + 32 * i + l] = (int8_t)(q2 - (h ? 0 : 4));
          }
      break;
    case T_IQ2_XS: case T_IQ2_S: case T_IQ3_XXS: case T_IQ3_S:
      /* signed code-book magnitudes, group (ib, il) of eight values as in oracle_dequantize */
      for (int ib = 0; ib < 8; ++ib)
        for (int il = 0; il < 4; ++il) {
          uint64_t grid;
          uint32_t signs;
          if (type == T_IQ2_XS) {
            uint32_t q = rd16(blk + 2 + 2 * (4 * ib + il));
            grid = gguf_b200_iq2xs_grid[q & 511];
            signs = gguf_b200_ksigns_iq2xs[q >> 9];
          } else if (type == T_IQ2_S) {
            grid = gguf_b200_iq2s_grid[blk[2 + 4 * ib + il] | (((uint32_t)blk[66 + ib] << (8 - 2 * il)) & 0x300)];
            signs = blk[2 + 32 + 4 * ib + il];
          } else if (type == T_IQ3_XXS) {
            const uint8_t* q3 = blk + 2 + 8 * ib;
            const uint8_t* g = blk + 2 + 64 + 4 * ib;
            uint32_t aux32 = (uint32_t)g[0] | ((uint32_t)g[1] << 8) | ((uint32_t)g[2] << 16) | ((uint32_t)g[3] << 24);
            grid = (uint64_t)gguf_b200_iq3xxs_grid[q3[2 * il]] | ((uint64_t)gguf_b200_iq3xxs_grid[q3[2 * il + 1]] << 32);
            signs = gguf_b200_ksigns_iq2xs[(aux32 >> (7 * il)) & 127];
          } else {
            const uint8_t* qs = blk + 2 + 8 * ib;
            uint32_t qh = blk[66 + ib];
            grid = (uint64_t)gguf_b200_iq3s_grid[qs[2 * il] | ((qh << (8 - 2 * il)) & 256)] |
                   ((uint64_t)gguf_b200_iq3s_grid[qs[2 * il + 1] | ((qh << (7 - 2 * il)) & 256)] << 32);
            signs = blk[74 + 4 * ib + il];
          }
          for (int j = 0; j < 8; ++j) {
            int g = (int)((grid >> (8 * j)) & 0xff);
            w[32 * ib + 8 * il + j] = (int8_t)(((signs >> j) & 1) ? -g : g);
          }
        }
      break;
    case T_IQ1_S: case T_IQ1_M:
      /* code-book values q in {0,1,2} (the "- 1 +- 1/8" enters through the activation sums) */
      for (int ib = 0; ib < 8; ++ib)
        for (int il = 0; il < 4; ++il) {
          uint32_t g;
          if (type == T_IQ1_S) {
            uint32_t qh = rd16(blk + 34 + 2 * ib);
            g = gguf_b200_iq1s_grid[blk[2 + 4 * ib + il] | (((qh >> (3 * il)) & 7) << 8)];
          } else {
            uint32_t qh = blk[32 + 2 * ib + il / 2];
            g = gguf_b200_iq1s_grid[blk[4 * ib + il] | (((qh >> (4 * (il % 2))) & 7) << 8)];
          }
          for (int j = 0; j < 8; ++j) w[32 * ib + 8 * il + j] = (int8_t)((g >> (8 * (j & 3) + 4 * (j >> 2))) & 0xf);
        }
      break;
  }
}

/* Dot product of one weight block with the aligned q8_1 block(s) y (36-byte blocks).
 * mmq = 0: the GEMV formulas (vec_dot_*_q8_1, vecdotq.cuh:493-509, 852-867, 1159-1202,
 *          1417-1441, 1531-1552, 1791-1812);
 * mmq = 1: the tiled-kernel formulas (vec_dot_*_q8_1_mul_mat, vecdotq.cuh:552-571, 912-921,
 *          1267-1277 with impl :353-379, 1518-1529), which differ for Q4_K: the min term
 *          uses the stored fp16 sum of the unquantized activations instead of d8*sum(q8). */
static double block_dot(const uint8_t* blk, int type, const uint8_t* y, int mmq) {
  int8_t w[QK_K];
  unpack_codes(blk, type, w);
  const int nsub = oracle_block_size(type) / 32;
  double acc = 0.0;
  switch (type) {
    case T_Q4_0: { /* d4 * (sumi*d8 - 8*s8), vec_dot_q4_0_q8_1_impl vecdotq.cuh:46-66 */
      double d4 = h2f(rd16(blk)), d8 = h2f(rd16(y)), s8 = h2f(rd16(y + 2));
      acc = d4 * (idot(w, (const int8_t*)y + 4, 32) * d8 - 8.0 * s8);
    } break;
    case T_Q8_0: { /* d8_0*d8_1*sumi, vecdotq.cuh:165-177 */
      acc = (double)h2f(rd16(blk)) * h2f(rd16(y)) * idot(w, (const int8_t*)y + 4, 32);
    } break;
    case T_Q4_K: { /* vecdotq.cuh:328-351 (GEMV) / :353-379 (tiled) */
      double d = h2f(rd16(blk)), dmin = h2f(rd16(blk + 2)), sd = 0, sm = 0;
      for (int g = 0; g < nsub; ++g) {
        int sc, m;
        scale_min_k4(g, blk + 4, &sc, &m);
        const uint8_t* yb = y + 36 * g;
        const int8_t* q8 = (const int8_t*)yb + 4;
        double d8 = h2f(rd16(yb)), s8 = h2f(rd16(yb + 2));
        sd += d8 * (double)(idot(w + 32 * g, q8, 32) * sc);
        if (mmq) {
          sm += s8 * m;
        } else {
          int sq = 0;
          for (int j = 0; j < 32; ++j) sq += q8[j];
          sm += d8 * (double)(sq * m);
        }
      }
      acc = d * sd - dmin * sm;
    } break;
    case T_Q6_K: { /* d * sum d8*(dot16*sc), vecdotq.cuh:447-491 */
      double d = h2f(rd16(blk + 208)), sf = 0;
      const int8_t* sc = (const int8_t*)(blk + 192);
      for (int g = 0; g < nsub; ++g) {
        const uint8_t* yb = y + 36 * g;
        const int8_t* q8 = (const int8_t*)yb + 4;
        double d8 = h2f(rd16(yb));
        sf += d8 * (double)(idot(w + 32 * g, q8, 16) * sc[2 * g] + idot(w + 32 * g + 16, q8 + 16, 16) * sc[2 * g + 1]);
      }
      acc = d * sf;
    } break;
    case T_IQ2_XXS: { /* d*(0.5+s)*d8*0.25*sumi, vecdotq.cuh:1531-1552 */
      double d = h2f(rd16(blk));
      for (int g = 0; g < nsub; ++g) {
        const uint8_t* yb = y + 36 * g;
        uint32_t s = blk[2 + 8 * g + 7] >> 4;
        acc += d * (0.5 + s) * h2f(rd16(yb)) * 0.25 * idot(w + 32 * g, (const int8_t*)yb + 4, 32);
      }
    } break;
    case T_Q2_K: { /* d * sum d8*(dot16*(sc&15)) - dmin * sum d8*((sc>>4)*sum16(q8)), vecdotq.cuh:204-232, 923-944 */
      double d = h2f(rd16(blk + 80)), dmin = h2f(rd16(blk + 82)), sd = 0, sm = 0;
      for (int g = 0; g < nsub; ++g) {
        const uint8_t* yb = y + 36 * g;
        const int8_t* q8 = (const int8_t*)yb + 4;
        double d8 = h2f(rd16(yb));
        for (int h = 0; h < 2; ++h) {
          int sc = blk[2 * g + h], sq = 0;
          for (int j = 0; j < 16; ++j) sq += q8[16 * h + j];
          sd += d8 * (double)(idot(w + 32 * g + 16 * h, q8 + 16 * h, 16) * (sc & 0xF));
          sm += d8 * (double)((sc >> 4) * sq);
        }
      }
      acc = d * sd - dmin * sm;
    } break;
    case T_Q3_K: { /* d * sum d8*(dot16*(sc6-32)), vecdotq.cuh:269-300, 1024-1048 */
      double d = h2f(rd16(blk + 108)), sf = 0;
      const uint8_t* sc = blk + 96;
      for (int g = 0; g < nsub; ++g) {
        const uint8_t* yb = y + 36 * g;
        const int8_t* q8 = (const int8_t*)yb + 4;
        double d8 = h2f(rd16(yb));
        for (int h = 0; h < 2; ++h) {
          int j = 2 * g + h;
          int s6 = (((sc[j % 8] >> (4 * (j / 8))) & 0xF) | (((sc[8 + j % 4] >> (2 * (j / 4))) & 3) << 4)) - 32;
          sf += d8 * (double)(idot(w + 32 * g + 16 * h, q8 + 16 * h, 16) * s6);
        }
      }
      acc = d * sf;
    } break;
    case T_IQ2_XS: case T_IQ2_S: { /* d*d8*0.25*((0.5+ls1)*sumi1 + (0.5+ls2)*sumi2), vecdotq.cuh:1554-1620 */
      double d = h2f(rd16(blk));
      const uint8_t* sc = blk + (type == T_IQ2_XS ? 66 : 74);
      for (int g = 0; g < nsub; ++g) {
        const uint8_t* yb = y + 36 * g;
        const int8_t* q8 = (const int8_t*)yb + 4;
        acc += d * h2f(rd16(yb)) * 0.25 * ((0.5 + (sc[g] & 0xf)) * idot(w + 32 * g, q8, 16) + (0.5 + (sc[g] >> 4)) * idot(w + 32 * g + 16, q8 + 16, 16));
      }
    } break;
    case T_IQ3_XXS: case T_IQ3_S: { /* d*(0.5+s)*d8*0.5*sumi, vecdotq.cuh:1622-1672 */
      double d = h2f(rd16(blk));
      for (int g = 0; g < nsub; ++g) {
        const uint8_t* yb = y + 36 * g;
        uint32_t s = type == T_IQ3_XXS ? (uint32_t)(blk[2 + 64 + 4 * g + 3] >> 4) : (uint32_t)((blk[106 + g / 2] >> (4 * (g % 2))) & 0xf);
        acc += d * (0.5 + s) * h2f(rd16(yb)) * 0.5 * idot(w + 32 * g, (const int8_t*)yb + 4, 32);
      }
    } break;
    case T_IQ1_S: { /* d*(2s+1) * (d8*sumi + s8*delta), vecdotq.cuh:1674-1704 */
      double d = h2f(rd16(blk));
      for (int g = 0; g < nsub; ++g) {
        const uint8_t* yb = y + 36 * g;
        uint32_t qh = rd16(blk + 34 + 2 * g);
        double delta = (qh & 0x8000) ? -1.0 - 0.125 : -1.0 + 0.125;
        acc += d * (double)(2 * ((qh >> 12) & 7) + 1) * (h2f(rd16(yb)) * idot(w + 32 * g, (const int8_t*)yb + 4, 32) + h2f(rd16(yb + 2)) * delta);
      }
    } break;
    case T_IQ1_M: { /* d*d8 * sum over the two halves of (sumi + delta*sum(q8)) * (2s+1), vecdotq.cuh:1706-1750 */
      uint32_t sc0 = rd16(blk + 48), sc1 = rd16(blk + 50), sc2 = rd16(blk + 52), sc3 = rd16(blk + 54);
      double d = h2f((uint16_t)((sc0 >> 12) | ((sc1 >> 8) & 0x00f0) | ((sc2 >> 4) & 0x0f00) | (sc3 & 0xf000)));
      for (int g = 0; g < nsub; ++g) {
        const uint8_t* yb = y + 36 * g;
        const int8_t* q8 = (const int8_t*)yb + 4;
        uint32_t tmp = rd16(blk + 48 + 2 * (g / 2)) >> (6 * (g % 2));
        double part = 0;
        for (int h = 0; h < 2; ++h) {      /* halves of 16 values, each with its own 3-bit scale */
          double sumf = 0;
          for (int l = 0; l < 2; ++l) {    /* groups of 8 values, each with its own delta bit */
            uint32_t qhl = blk[32 + 2 * g + h] >> (4 * l);
            double delta = (qhl & 0x08) ? -1.0 - 0.125 : -1.0 + 0.125;
            int sumy = 0;
            for (int j = 0; j < 8; ++j) sumy += q8[16 * h + 8 * l + j];
            sumf += delta * sumy;
          }
          part += (idot(w + 32 * g + 16 * h, q8 + 16 * h, 16) + sumf) * (double)(2 * ((tmp >> (3 * h)) & 7) + 1);
        }
        acc += d * h2f(rd16(yb)) * part;
      }
    } break;
    case T_IQ4_XS: { /* d*(ls-32)*d8*(sumi1+sumi2), vecdotq.cuh:1791-1812 */
      double d = h2f(rd16(blk));
      for (int g = 0; g < nsub; ++g) {
        const uint8_t* yb = y + 36 * g;
        acc += d * iq4xs_ls(blk, g) * h2f(rd16(yb)) * idot(w + 32 * g, (const int8_t*)yb + 4, 32);
      }
    } break;
    case T_Q4_1:   /* sumi * h(d4*d8) + h(m4*s8): both products in half (__hmul2), vecdotq.cuh:72-96 */
    case T_Q5_1: { /* the same with 5-bit codes, vecdotq.cuh:134-163 */
      uint16_t d = rd16(blk), m = rd16(blk + 2);
      acc = (double)idot(w, (const int8_t*)y + 4, 32) * h2f(hmul(d, rd16(y))) + h2f(hmul(m, rd16(y + 2)));
    } break;
    case T_Q5_0: { /* d5 * (sumi*d8 - 16*s8), vecdotq.cuh:101-129.  The tiled kernel folds the -16 into
                      the codes and drops the s8 term (load_tiles_q5_0 + vec_dot_q8_0_q8_1_impl). */
      double d5 = h2f(rd16(blk)), d8 = h2f(rd16(y)), s8 = h2f(rd16(y + 2));
      if (mmq) {
        int sumi = 0;
        for (int j = 0; j < 32; ++j) sumi += (w[j] - 16) * ((const int8_t*)y + 4)[j];
        acc = d5 * d8 * sumi;
      } else {
        acc = d5 * (idot(w, (const int8_t*)y + 4, 32) * d8 - 16.0 * s8);
      }
    } break;
    case T_IQ4_NL: /* d * d8 * (sumi1 + sumi2), vecdotq.cuh:1766-1789 */
      acc = (double)h2f(rd16(blk)) * h2f(rd16(y)) * idot(w, (const int8_t*)y + 4, 32);
      break;
    case T_Q5_K: { /* vecdotq.cuh:386-413 (GEMV) / :415-445 (tiled), as Q4_K with 5-bit codes */
      double d = h2f(rd16(blk)), dmin = h2f(rd16(blk + 2)), sd = 0, sm = 0;
      for (int g = 0; g < nsub; ++g) {
        int sc, m;
        scale_min_k4(g, blk + 4, &sc, &m);
        const uint8_t* yb = y + 36 * g;
        const int8_t* q8 = (const int8_t*)yb + 4;
        double d8 = h2f(rd16(yb)), s8 = h2f(rd16(yb + 2));
        sd += d8 * (double)(idot(w + 32 * g, q8, 32) * sc);
        if (mmq) {
          sm += s8 * m;
        } else {
          int sq = 0;
          for (int j = 0; j < 32; ++j) sq += q8[j];
          sm += d8 * (double)(sq * m);
        }
      }
      acc = d * sd - dmin * sm;
    } break;
  }
  return acc;
}

/* ------------------------------------------------------------------ */
/* matmul entry points                                                 */
/* ------------------------------------------------------------------ */

/* Y[m, n] = sum over blocks of row n of block_dot(W block, q8_1 blocks of vector m).
 * Covers ggml_mul_mat_vec_a8 (mmq=0; gguf_kernel.cu:104-218 + mmvq.cuh:2-41) and
 * ggml_mul_mat_a8 (mmq=1; gguf_kernel.cu:220-290 + mmq.cuh:2-104): both quantize X to q8_1
 * first.  xq = output of oracle_quantize_q8_1 (row stride Kpad/32 blocks).
 * y64 receives the unrounded value; out (may be NULL) the value stored as out_dt. */
int oracle_matmul_a8(const uint8_t* w, int type, const uint8_t* xq, double* y64, void* out, int out_dt,
                     int64_t M, int64_t N, int64_t K, int mmq) {
  const int ts = oracle_type_size(type), bs = oracle_block_size(type);
  if (!ts || K % bs) return -1;
  const int64_t bpr = K / bs, qrow = oracle_q8_1_row_bytes(K);
  for (int64_t m = 0; m < M; ++m)
    for (int64_t n = 0; n < N; ++n) {
      double acc = 0;
      for (int64_t b = 0; b < bpr; ++b)
        acc += block_dot(w + (n * bpr + b) * ts, type, xq + m * qrow + b * (bs / 32) * 36, mmq);
      if (y64) y64[m * N + n] = acc;
      if (out) store_f(out, out_dt, m * N + n, (float)acc);
    }
  return 0;
}

/* ggml_moe_a8 (gguf_kernel.cu:292-393 + moe_q, moe.cuh:5-129).  For every position p of
 * sorted_token_ids below num_tokens_post_padded whose id t = sorted[p] is a real slot
 * (t < tokens*top_k): activation row t/top_k (moe.cuh:64), expert expert_ids[p/block]
 * (moe.cuh:32), output row t (moe.cuh:115-126).  Rows never written stay zero
 * (new_zeros, gguf_kernel.cu:301-302).  Experts outside [0,255] are skipped (moe.cuh:33).
 * Arithmetic = the tiled-kernel formulas (mmq=1). */
int oracle_moe_a8(const uint8_t* w, int type, const uint8_t* xq, double* y64, void* out, int out_dt,
                  const int32_t* sorted_ids, int64_t n_sorted, const int32_t* expert_ids, int32_t n_post_pad,
                  int block, int64_t expert_stride_bytes, int64_t tokens, int64_t top_k, int64_t N, int64_t K) {
  const int ts = oracle_type_size(type), bs = oracle_block_size(type);
  if (!ts || K % bs) return -1;
  const int64_t bpr = K / bs, qrow = oracle_q8_1_row_bytes(K), rows = tokens * top_k;
  for (int64_t i = 0; i < rows * N; ++i) {
    if (y64) y64[i] = 0;
    if (out) store_f(out, out_dt, i, 0.0f);
  }
  for (int64_t p = 0; p < n_sorted && p < n_post_pad; ++p) {
    const int64_t t = sorted_ids[p];
    const int e = expert_ids[p / block];
    if (t < 0 || t >= rows || e < 0 || e > 255) continue;
    const uint8_t* we = w + e * expert_stride_bytes;
    const uint8_t* xr = xq + (t / top_k) * qrow;
    for (int64_t n = 0; n < N; ++n) {
      double acc = 0;
      for (int64_t b = 0; b < bpr; ++b) acc += block_dot(we + (n * bpr + b) * ts, type, xr + b * (bs / 32) * 36, 1);
      if (y64) y64[t * N + n] = acc;
      if (out) store_f(out, out_dt, t * N + n, (float)acc);
    }
  }
  return 0;
}

/* ggml_moe_a8_vec (gguf_kernel.cu:395-530 + moe_vec_q, moe_vec.cuh:3-53): output row
 * s = token*top_k + k uses expert topk_ids[s] and activation row s/top_k, GEMV formulas. */
int oracle_moe_a8_vec(const uint8_t* w, int type, const uint8_t* xq, double* y64, void* out, int out_dt,
                      const int32_t* topk_ids, int64_t tokens, int64_t top_k, int64_t N, int64_t K) {
  const int ts = oracle_type_size(type), bs = oracle_block_size(type);
  if (!ts || K % bs) return -1;
  const int64_t bpr = K / bs, qrow = oracle_q8_1_row_bytes(K);
  for (int64_t s = 0; s < tokens * top_k; ++s) {
    const uint8_t* we = w + (int64_t)topk_ids[s] * N * bpr * ts;
    const uint8_t* xr = xq + (s / top_k) * qrow;
    for (int64_t n = 0; n < N; ++n) {
      double acc = 0;
      for (int64_t b = 0; b < bpr; ++b) acc += block_dot(we + (n * bpr + b) * ts, type, xr + b * (bs / 32) * 36, 0);
      if (y64) y64[s * N + n] = acc;
      if (out) store_f(out, out_dt, s * N + n, (float)acc);
    }
  }
  return 0;
}

/* Dense fp32 dot of dequantized weights with raw activations: the arithmetic of the
 * reference's dequantize-then-matmul route for IQ types at larger batches
 * (quantization/linear.py:50-54).  wd = fp32 view of the dequantized weights [N,K]. */
int oracle_dense_matmul(const float* wd, const void* x, int x_dt, double* y64, int64_t M, int64_t N, int64_t K) {
  for (int64_t m = 0; m < M; ++m)
    for (int64_t n = 0; n < N; ++n) {
      double acc = 0;
      for (int64_t k = 0; k < K; ++k) acc += (double)wd[n * K + k] * load_act(x, x_dt, m * K + k);
      y64[m * N + n] = acc;
    }
  return 0;
}
