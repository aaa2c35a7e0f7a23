// Fused dequant-GEMV for decode:  Y[m, n] = sum_k dequant(W)[n, k] * q8_1(X)[m, k]
// (reference: ggml_mul_mat_vec_a8, vllm_gguf_plugin/csrc/gguf/gguf_kernel.cu:104-218; kernel
// mul_mat_vec_q, mmvq.cuh:2-41; per-type block dot products vec_dot_*_q8_1, vecdotq.cuh:493-509,
// 852-867, 1159-1202, 1417-1441, 1531-1552, 1791-1812).
//
// The op is bound by reading the packed weights once from HBM, so the kernel is built
// around keeping many bytes in flight per SM rather than around the arithmetic:
//  * each warp owns whole output rows and streams a row (or a row segment of <= `payload`
//    bytes) into its private ring of shared-memory stages with ONE 1-D bulk copy (TMA) per
//    segment, completion signalled on an mbarrier; `stages`-1 copies are always outstanding
//    per warp, 8 warps per CTA, 2 CTAs per SM;
//  * rows of Q8_0 / Q4_0 / Q6_K / IQ2_XXS are only 2-byte aligned, bulk copies need 16: the
//    copy starts at the row address rounded down to 16 bytes and the decoder indexes from the
//    remainder with funnel shifts;
//  * the q8_1 activations of up to MT vectors are staged once per CTA in shared memory
//    (int8 codes + float2 {d, sum} per 32), so the weights are read once for all MT vectors --
//    the reference re-reads them per vector (grid.y = M, mmvq.cuh:45-49);
//  * lanes split a segment in units of 32..64 values, integer dot products use dp4a, the
//    per-lane fp32 partial sums are combined with a shuffle butterfly.
// The IQ2_XXS grid and an expanded sign-mask table live in shared memory because lanes index
// them with unrelated values.
//
// All waits are bounded; on expiry the kernel sets *status and returns.
#include "common.cuh"
#include "kernels.h"
#include "tables.cuh"

namespace gguf_b200 {

constexpr int GEMV_WARPS = 8;
constexpr int STAGE_SLACK = 32;  // 16 for the rounded-down start + 16 for the rounded-up end

template <int TYPE> struct GemvTraits;
template <> struct GemvTraits<T_Q4_0>    { static constexpr int UPB = 1; };  // units (lane work items) per block
template <> struct GemvTraits<T_Q8_0>    { static constexpr int UPB = 1; };
template <> struct GemvTraits<T_Q4_K>    { static constexpr int UPB = 4; };  // 64 values each
template <> struct GemvTraits<T_Q6_K>    { static constexpr int UPB = 4; };  // 64 values each
template <> struct GemvTraits<T_IQ2_XXS> { static constexpr int UPB = 8; };  // 32 values each
template <> struct GemvTraits<T_IQ4_XS>  { static constexpr int UPB = 8; };

// Activations in shared memory.  The int8 codes are stored in 16-byte chunks (chunk c = values
// 16c..16c+15) at the swizzled position c ^ ((c >> 3) & 7): lanes of a warp read chunks that are
// 1, 2 or 4 apart (one unit per lane), and the swizzle spreads any such stride over all eight
// 16-byte bank groups, so a 128-bit load costs its minimum of four wavefronts.
struct XView {
  const uint4* qs;     // vector m at qs + m*(kpad/16)
  const float2* ds;    // {d, sum} per 32 values, vector m at ds + m*nb
  int chunks, nb;      // kpad/16, kpad/32
};

__device__ __forceinline__ int swz(int c) { return c ^ ((c >> 3) & 7); }
__device__ __forceinline__ void load_x32(const XView& x, int m, int g, uint32_t (&u)[8]) {
  const uint4* p = x.qs + (size_t)m * x.chunks;
  const uint4 a = p[swz(2 * g)], b = p[swz(2 * g + 1)];
  u[0] = a.x; u[1] = a.y; u[2] = a.z; u[3] = a.w;
  u[4] = b.x; u[5] = b.y; u[6] = b.z; u[7] = b.w;
}
__device__ __forceinline__ int dp4a8(const uint32_t (&w)[8], const uint32_t (&u)[8]) {
  int s = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) s = __dp4a((int)w[i], (int)u[i], s);
  return s;
}
// unsigned bytes (weights) times signed bytes (activations)
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
// n consecutive 32-bit words from a 2-byte aligned shared address
template <int N> __device__ __forceinline__ void lds_words_a2(const uint8_t* p, uint32_t (&w)[N]) { lds_words_unaligned<N>(p, w); }

struct Tables {
  const uint2* grid;    // IQ2_XXS: 256 x 8 magnitudes
  const uint2* smask;   // IQ2_XXS: 128 x 8 byte masks (0xFF where the value is negative)
  uint32_t kv[4];       // IQ4_XS: the 16 levels packed four per register
};

// ---- one unit of work per lane --------------------------------------------------------

template <int TYPE, int MT> struct Unit;

template <int MT> struct Unit<T_Q8_0, MT> {   // sum_i d*d8*dot, vec_dot_q8_0_q8_1
  static __device__ __forceinline__ void run(const uint8_t* blk, int, int g, const XView& x, const Tables&, int mc, float (&acc)[MT]) {
    const float d = lds_half_as_float(blk);
    uint32_t w[8];
    lds_words_a2<8>(blk + 2, w);
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      if (m < mc) {
        uint32_t u[8];
        load_x32(x, m, g, u);
        acc[m] += d * x.ds[m * x.nb + g].x * (float)dp4a8(w, u);
      }
    }
  }
};

template <int MT> struct Unit<T_Q4_0, MT> {   // d4*(sumi*d8 - 8*s8), vec_dot_q4_0_q8_1
  static __device__ __forceinline__ void run(const uint8_t* blk, int, int g, const XView& x, const Tables&, int mc, float (&acc)[MT]) {
    const float d = lds_half_as_float(blk);
    uint32_t q[4];
    lds_words_a2<4>(blk + 2, q);
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      if (m < mc) {
        uint32_t u[8];
        load_x32(x, m, g, u);
        int lo = 0, hi = 0;  // hi accumulates 16 * (high-nibble dot): the nibbles stay in place
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          lo = dp4a_us(q[i] & 0x0F0F0F0Fu, u[i], lo);      // values 4i..4i+3
          hi = dp4a_us(q[i] & 0xF0F0F0F0u, u[4 + i], hi);  // values 16+4i..
        }
        const float2 ds = x.ds[m * x.nb + g];
        acc[m] += d * ((float)(lo + (hi >> 4)) * ds.x - 8.0f * ds.y);
      }
    }
  }
};

template <int MT> struct Unit<T_Q4_K, MT> {   // unit p = 64 values: sub-blocks 2p (low nibbles) and 2p+1
  static __device__ __forceinline__ void run(const uint8_t* blk, int p, int g0, const XView& x, const Tables&, int mc, float (&acc)[MT]) {
    const uint4 hdr = *reinterpret_cast<const uint4*>(blk);  // dm | scales[0..3] | [4..7] | [8..11]
    const __half2 dm = *reinterpret_cast<const __half2*>(&hdr.x);
    const float d = __low2float(dm), dmin = __high2float(dm);
    // 6-bit (scale, min) of sub-blocks j = 2p, 2p+1 (get_scale_min_k4), both selected without a branch:
    // j < 4: sc = b[j] & 63, m = b[j+4] & 63;  j >= 4: sc = (b[j+4] & 15) | (b[j-4] >> 6) << 4, m = (b[j+4] >> 4) | (b[j] >> 6) << 4
    const int sh = 16 * (p & 1);
    const uint32_t a = hdr.y >> sh, b = hdr.z >> sh, c = hdr.w >> sh;  // low 16 bits: the byte pair of interest
    const bool low = p < 2;
    const uint32_t sc2 = low ? (a & 0x3F3Fu) : ((c & 0x0F0Fu) | ((a >> 2) & 0x3030u));
    const uint32_t mn2 = low ? (b & 0x3F3Fu) : (((c >> 4) & 0x0F0Fu) | ((b >> 2) & 0x3030u));
    const int sc0 = sc2 & 0xFF, sc1 = (sc2 >> 8) & 0xFF;
    const float m0 = (float)(mn2 & 0xFF), m1 = (float)((mn2 >> 8) & 0xFF);
    const uint4* qp = reinterpret_cast<const uint4*>(blk + 16 + 32 * p);
    const uint4 qa = qp[0], qb = qp[1];
    const uint32_t q[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
    const int g = g0 + 2 * p;
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      if (m < mc) {
        uint32_t u0[8], u1[8];
        load_x32(x, m, g, u0);
        load_x32(x, m, g + 1, u1);
        int dot0 = 0, dot1 = 0;  // dot1 = 16 * (high-nibble dot)
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          dot0 = dp4a_us(q[i] & 0x0F0F0F0Fu, u0[i], dot0);
          dot1 = dp4a_us(q[i] & 0xF0F0F0F0u, u1[i], dot1);
        }
        const float4 ds = *reinterpret_cast<const float4*>(&x.ds[m * x.nb + g]);  // d8_0, s_0, d8_1, s_1
        // ds.y / ds.w hold d8*sum(q8) for this entry point (the GEMV recomputes the sum from the codes)
        acc[m] += d * (ds.x * (float)(dot0 * sc0) + ds.z * (float)((dot1 >> 4) * sc1)) - dmin * (ds.y * m0 + ds.w * m1);
      }
    }
  }
};

template <int MT> struct Unit<T_Q6_K, MT> {   // unit u: half ip = u>>1, column half h = u&1 -> groups 4ip+h and 4ip+2+h
  static __device__ __forceinline__ void run(const uint8_t* blk, int u4, int g0, const XView& x, const Tables&, int mc, float (&acc)[MT]) {
    const int ip = u4 >> 1, h = u4 & 1;
    uint32_t ql[8], qh[8];
    lds_words_a2<8>(blk + 64 * ip + 32 * h, ql);
    lds_words_a2<8>(blk + 128 + 32 * ip, qh);
    const int8_t* scp = reinterpret_cast<const int8_t*>(blk + 192 + 8 * ip + 2 * h);
    const int sa0 = scp[0], sa1 = scp[1], sb0 = scp[4], sb1 = scp[5];
    const float d = lds_half_as_float(blk + 208);
    uint32_t va[8], vb[8];
    const int s2 = 2 * h;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t hh = qh[i] >> s2;  // bits 0-1 of each byte: group A, bits 4-5: group B
      const uint32_t a = (ql[i] & 0x0F0F0F0Fu) | ((hh << 4) & 0x30303030u);
      const uint32_t b = ((ql[i] >> 4) & 0x0F0F0F0Fu) | (hh & 0x30303030u);
      va[i] = (a + 0x60606060u) ^ 0x80808080u;  // per byte: code - 32 as int8 (no carries: code <= 63)
      vb[i] = (b + 0x60606060u) ^ 0x80808080u;
    }
    const int ga = g0 + 4 * ip + h, gb = ga + 2;
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      if (m < mc) {
        uint32_t ua[8], ub[8];
        load_x32(x, m, ga, ua);
        load_x32(x, m, gb, ub);
        int a0 = 0, a1 = 0, b0 = 0, b1 = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          a0 = __dp4a((int)va[i], (int)ua[i], a0);
          a1 = __dp4a((int)va[4 + i], (int)ua[4 + i], a1);
          b0 = __dp4a((int)vb[i], (int)ub[i], b0);
          b1 = __dp4a((int)vb[4 + i], (int)ub[4 + i], b1);
        }
        acc[m] += d * (x.ds[m * x.nb + ga].x * (float)(a0 * sa0 + a1 * sa1) +
                       x.ds[m * x.nb + gb].x * (float)(b0 * sb0 + b1 * sb1));
      }
    }
  }
};

template <int MT> struct Unit<T_IQ4_XS, MT> {   // unit ib = 32 values
  // Levels of four 4-bit indices (low 16 bits of q3, bit 3 of each cleared; sel = which table half):
  // two byte-permutes pick from levels 0-7 and 8-15 by the low three bits, a third merges them.
  static __device__ __forceinline__ uint32_t lut4(uint32_t q3, uint32_t sel, const Tables& t) {
    return __byte_perm(__byte_perm(t.kv[0], t.kv[1], q3), __byte_perm(t.kv[2], t.kv[3], q3), sel);
  }
  static __device__ __forceinline__ void run(const uint8_t* blk, int ib, int g0, const XView& x, const Tables& t, int mc, float (&acc)[MT]) {
    const uint2 hdr = *reinterpret_cast<const uint2*>(blk);  // d | scales_h | scales_l[4]
    const float d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xffff)));
    const int ls = (int)(((hdr.y >> (4 * ib)) & 0xF) | ((((hdr.x >> 16) >> (2 * ib)) & 3) << 4)) - 32;
    const uint2* qp = reinterpret_cast<const uint2*>(blk + 8 + 16 * ib);
    const uint2 qa = qp[0], qb = qp[1];
    const uint32_t q[4] = {qa.x, qa.y, qb.x, qb.y};
    uint32_t w[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      // the packed word is its own selector: nibbles (b0 lo, b0 hi, b1 lo, b1 hi | b2 ..) = values (4i, 16+4i, 4i+1, 17+4i | ..)
      const uint32_t q3 = q[i] & 0x77777777u;
      const uint32_t sel = ((q[i] & 0x88888888u) >> 1) | 0x32103210u;
      const uint32_t a = lut4(q3, sel, t), b = lut4(q3 >> 16, sel >> 16, t);
      w[i] = __byte_perm(a, b, 0x6420);       // values 4i..4i+3
      w[4 + i] = __byte_perm(a, b, 0x7531);   // values 16+4i..
    }
    const int g = g0 + ib;
    const float dl = d * (float)ls;
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      if (m < mc) {
        uint32_t u[8];
        load_x32(x, m, g, u);
        acc[m] += dl * x.ds[m * x.nb + g].x * (float)dp4a8(w, u);
      }
    }
  }
};

template <int MT> struct Unit<T_IQ2_XXS, MT> {   // unit ib = 32 values: 4 grid points + signs + 4-bit scale
  static __device__ __forceinline__ void run(const uint8_t* blk, int ib, int g0, const XView& x, const Tables& t, int mc, float (&acc)[MT]) {
    const float d = lds_half_as_float(blk);
    uint32_t q[2];
    lds_words_a2<2>(blk + 2 + 8 * ib, q);
    const uint32_t aux = q[1];
    uint32_t gp[8], gn[8];
#pragma unroll
    for (int il = 0; il < 4; ++il) {
      const uint2 gr = t.grid[(q[0] >> (8 * il)) & 0xFF];
      const uint2 sm = t.smask[(aux >> (7 * il)) & 127];
      gp[2 * il] = gr.x;
      gp[2 * il + 1] = gr.y;
      gn[2 * il] = gr.x & sm.x;
      gn[2 * il + 1] = gr.y & sm.y;
    }
    const int g = g0 + ib;
    const float dl = d * (0.5f + (float)(aux >> 28)) * 0.25f;
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      if (m < mc) {
        uint32_t u[8];
        load_x32(x, m, g, u);
        // sum g*s*q8 with s = +-1  ==  sum g*q8 - 2 * sum_{negative} g*q8
        const int sumi = dp4a8(gp, u) - 2 * dp4a8(gn, u);
        acc[m] += dl * x.ds[m * x.nb + g].x * (float)sumi;
      }
    }
  }
};

// ---- the kernel -----------------------------------------------------------------------

struct GemvParams {
  const uint8_t* w;       // packed weights, N rows of row_bytes
  int64_t w_bytes;        // total weight bytes (bulk copies never read past this rounded down to 16)
  const uint8_t* xq;      // SoA q8_1 activations of all M vectors
  int64_t m_total;        // number of vectors in xq
  int m0, mc;             // this launch handles vectors m0 .. m0+mc-1 (mc <= MT)
  void* y;                // [M][N]
  int64_t n, k;
  int bpr;                // blocks per row
  int seg_blocks, nseg;   // row segmentation
  int stages, stage_bytes;
  // MoE-vec mode (topk_ids != null): output row s uses weights of expert topk_ids[s], vector s/top_k
  const int32_t* topk_ids;
  int64_t n_slots, top_k, expert_rows, n_experts;
  int* status;
};

template <int TYPE, int MT, typename out_t>
__global__ void __launch_bounds__(GEMV_WARPS * 32, MT == 1 ? 3 : 2) gemv_kernel(const GemvParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int TS = BlockTraits<TYPE>::TS, QK = BlockTraits<TYPE>::QK, UPB = GemvTraits<TYPE>::UPB;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kpad = (int)round_up(p.k, 512), nb = kpad / 32;
  const bool moe = p.topk_ids != nullptr;

  // shared layout: [x codes MT*kpad][x scales MT*nb*8][tables][rings][barriers]
  uint4* s_xq = reinterpret_cast<uint4*>(smem);
  float2* s_xd = reinterpret_cast<float2*>(smem + (size_t)MT * kpad);
  uint8_t* cur = smem + (size_t)MT * kpad + (size_t)MT * nb * 8;
  Tables tb;
  tb.grid = nullptr;
  tb.smask = nullptr;
  if (TYPE == T_IQ2_XXS) {
    uint2* g = reinterpret_cast<uint2*>(cur);
    uint2* sm = g + 256;
    cur += 256 * 8 + 128 * 8;
    for (int i = threadIdx.x; i < 256; i += blockDim.x) {
      const uint64_t v = d_iq2xxs_grid[i];
      g[i] = make_uint2((uint32_t)v, (uint32_t)(v >> 32));
    }
    for (int i = threadIdx.x; i < 128; i += blockDim.x) {
      const uint32_t s = d_ksigns_iq2xs[i];
      uint32_t lo = 0, hi = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        lo |= ((s >> j) & 1u) ? (0xFFu << (8 * j)) : 0u;
        hi |= ((s >> (4 + j)) & 1u) ? (0xFFu << (8 * j)) : 0u;
      }
      sm[i] = make_uint2(lo, hi);
    }
    tb.grid = g;
    tb.smask = sm;
  }
  if (TYPE == T_IQ4_XS) {
    const uint32_t* kv = reinterpret_cast<const uint32_t*>(d_kvalues_iq4nl);
#pragma unroll
    for (int i = 0; i < 4; ++i) tb.kv[i] = kv[i];
  }
  uint8_t* ring = cur + (size_t)warp * p.stages * p.stage_bytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(cur + (size_t)GEMV_WARPS * p.stages * p.stage_bytes) + warp * p.stages;

  if (lane == 0)
    for (int s = 0; s < p.stages; ++s) mbar_init(&bars[s], 1);
  fence_barrier_init();
  __syncwarp();

  // Row ownership.  Dense: rows interleaved over all warps of the grid (the 8 warps of a CTA read
  // 8 consecutive rows).  MoE-vec: each warp owns a contiguous run, so its vector changes rarely.
  const int64_t total_rows = moe ? p.n_slots * p.n : p.n;
  const int64_t gwarps = (int64_t)gridDim.x * GEMV_WARPS;
  const int64_t gw = (int64_t)blockIdx.x * GEMV_WARPS + warp;
  const int64_t rpw = (total_rows + gwarps - 1) / gwarps;
  int64_t row0, row_step;
  int my_rows;
  if (moe) {
    int64_t c = total_rows - gw * rpw;
    my_rows = (int)(c < 0 ? 0 : (c > rpw ? rpw : c));
    row0 = gw * rpw;
    row_step = 1;
  } else {
    my_rows = gw < total_rows ? (int)((total_rows - gw + gwarps - 1) / gwarps) : 0;
    row0 = gw;
    row_step = gwarps;
  }
  const int64_t row_bytes = (int64_t)p.bpr * TS;
  const int64_t w_safe = p.w_bytes & ~int64_t(15);
  const uint32_t n32 = (uint32_t)p.n;

  // weight row of logical row r (MoE-vec: r = slot * N + n uses the slot's expert); -1 when the
  // slot's expert id is not in [0, n_experts): such rows are neither read nor written
  auto weight_row = [&](int64_t r) -> int64_t {
    if (!moe) return r;
    const uint32_t slot = (uint32_t)r / n32;
    const int64_t e = p.topk_ids[slot];
    if (e < 0 || e >= p.n_experts) return -1;
    return e * p.expert_rows + (int64_t)((uint32_t)r - slot * n32);
  };
  // Issue the bulk copy of (row iteration ri, segment seg) into stage st.  Lane 0 only.
  auto issue = [&](int ri, int seg, int st) {
    const int64_t wrow = weight_row(row0 + (int64_t)ri * row_step);
    const int b0 = seg * p.seg_blocks;
    const int nbk = min(p.seg_blocks, p.bpr - b0);
    const int64_t beg = wrow * row_bytes + (int64_t)b0 * TS, end = beg + (int64_t)nbk * TS;
    const int64_t abeg = beg & ~int64_t(15);
    int64_t aend = (end + 15) & ~int64_t(15);
    if (aend > w_safe) aend = w_safe;  // the (< 16 byte) tail past w_safe is fetched with plain loads by the consumer
    uint8_t* dst = ring + (size_t)st * p.stage_bytes;
    const uint32_t bytes = (wrow >= 0 && aend > abeg) ? (uint32_t)(aend - abeg) : 0u;
    if (bytes) {
      mbar_expect_tx(&bars[st], bytes);
      bulk_g2s(dst, p.w + abeg, bytes, &bars[st]);
    } else {
      mbar_arrive(&bars[st]);
    }
  };

  // producer cursor (row iteration, segment, stage), advanced one item at a time: no divisions
  int p_ri = 0, p_seg = 0, p_st = 0;
  auto advance_producer = [&]() {
    if (++p_seg == p.nseg) { p_seg = 0; ++p_ri; }
    if (++p_st == p.stages) p_st = 0;
  };
  for (int i = 0; i < p.stages - 1; ++i) {
    if (p_ri < my_rows) {
      if (lane == 0) issue(p_ri, p_seg, p_st);
      advance_producer();
    }
  }

  pdl_wait();  // the weight copies above are independent of earlier kernels; the activations are not
  // Stage the activations (dense mode: vectors m0..m0+mc-1, shared by all rows).
  XView xv;
  xv.qs = s_xq;
  xv.ds = s_xd;
  xv.chunks = kpad / 16;
  xv.nb = nb;
  if (!moe) {
    const uint4* src = reinterpret_cast<const uint4*>(p.xq + (size_t)p.m0 * kpad);
    const int cpv = kpad / 16;
    for (int i = threadIdx.x; i < p.mc * cpv; i += blockDim.x) {
      const int m = i / cpv, c = i - m * cpv;
      s_xq[m * cpv + swz(c)] = __ldg(src + i);
    }
    const float2* dsrc = reinterpret_cast<const float2*>(p.xq + (size_t)p.m_total * kpad) + (size_t)p.m0 * nb;
    for (int i = threadIdx.x; i < p.mc * nb; i += blockDim.x) s_xd[i] = __ldg(dsrc + i);
  }
  __syncthreads();

  float acc[MT];
#pragma unroll
  for (int m = 0; m < MT; ++m) acc[m] = 0.f;
  uint32_t cur_slot = 0xFFFFFFFFu;
  int c_st = 0;
  uint32_t c_phase = 0;

  for (int ri = 0; ri < my_rows; ++ri) {
    const int64_t r = row0 + (int64_t)ri * row_step;
    const int64_t wrow = weight_row(r);
    if (moe) {
      const uint32_t slot = (uint32_t)r / n32;
      if (slot != cur_slot) {  // this warp's activation vector changes: restage it into the warp's slice
        const int64_t tok = slot / (uint32_t)p.top_k;
        const uint4* src = reinterpret_cast<const uint4*>(p.xq + (size_t)tok * kpad);
        uint4* dst = s_xq + (size_t)warp * xv.chunks;
        __syncwarp();
        for (int i = lane; i < xv.chunks; i += 32) dst[swz(i)] = __ldg(src + i);
        const float2* dsrc = reinterpret_cast<const float2*>(p.xq + (size_t)p.m_total * kpad) + (size_t)tok * nb;
        for (int i = lane; i < nb; i += 32) s_xd[(size_t)warp * nb + i] = __ldg(dsrc + i);
        __syncwarp();
        cur_slot = slot;
      }
    }
    for (int seg = 0; seg < p.nseg; ++seg) {
      if (p_ri < my_rows) {  // keep stages-1 copies in flight
        if (lane == 0) issue(p_ri, p_seg, p_st);
        advance_producer();
      }
      if (!mbar_wait_bounded(&bars[c_st], c_phase)) {
        if (lane == 0) atomicExch(p.status, E_TIMEOUT);
        drain_pause();   // copies this warp still has in flight land before its CTA can retire
        return;
      }
      const int b0 = seg * p.seg_blocks;
      const int nbk = min(p.seg_blocks, p.bpr - b0);
      const int64_t beg = wrow * row_bytes + (int64_t)b0 * TS;
      uint8_t* stage = ring + (size_t)c_st * p.stage_bytes;
      const uint8_t* data = stage + (beg & 15);
      {  // tail bytes the bulk copy was not allowed to touch
        const int64_t end = beg + (int64_t)nbk * TS;
        if (wrow >= 0 && end > w_safe) {
          const int64_t abeg = beg & ~int64_t(15);
          for (int64_t o = w_safe + lane; o < end; o += 32) stage[o - abeg] = p.w[o];
          __syncwarp();
        }
      }
      const int units = wrow >= 0 ? nbk * UPB : 0;
      const int g_seg = b0 * (QK / 32);
      if (moe) {
        XView xw = xv;  // one vector per warp, stored in slice `warp`
        xw.qs = s_xq + (size_t)warp * xv.chunks;
        xw.ds = s_xd + (size_t)warp * nb;
        float a1[1] = {acc[0]};
        for (int u = lane; u < units; u += 32) {
          const int b = u / UPB;
          Unit<TYPE, 1>::run(data + b * TS, u - b * UPB, g_seg + b * (QK / 32), xw, tb, 1, a1);
        }
        acc[0] = a1[0];
      } else {
        for (int u = lane; u < units; u += 32) {
          const int b = u / UPB;
          Unit<TYPE, MT>::run(data + b * TS, u - b * UPB, g_seg + b * (QK / 32), xv, tb, p.mc, acc);
        }
      }
      __syncwarp();  // all lanes are done with this stage before lane 0 refills it
      if (++c_st == p.stages) { c_st = 0; c_phase ^= 1u; }
    }
    out_t* y = static_cast<out_t*>(p.y);
    if (moe) {
      const float v = warp_sum(acc[0]);
      if (lane == 0 && wrow >= 0) y[r] = from_float<out_t>(v);
      acc[0] = 0.f;
    } else {
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        const float v = warp_sum(acc[m]);
        if (lane == m && m < p.mc) y[(int64_t)(p.m0 + m) * p.n + r] = from_float<out_t>(v);
        acc[m] = 0.f;
      }
    }
  }
}

// ---- host side ------------------------------------------------------------------------

int64_t q8_soa_bytes(int64_t M, int64_t K) {
  const int64_t kpad = round_up(K, 512);
  return M * kpad + M * (kpad / 32) * 8;
}

struct GemvPlan {
  int seg_blocks, nseg, stages, stage_bytes, mt;
  size_t smem;
};

static int gemv_tune_int(const char* name, int dflt) {
  const char* v = getenv(name);
  return v && *v ? atoi(v) : dflt;
}

static GemvPlan make_plan(int type, int64_t K, int64_t M, bool moe) {
  static const int payload_env = gemv_tune_int("GGUF_B200_GEMV_PAYLOAD", 2304);
  static const int stages_env = gemv_tune_int("GGUF_B200_GEMV_STAGES", 3);
  const int ts = type_size(type), qk = block_size(type);
  const int bpr = (int)(K / qk);
  const int upb = (type == T_Q4_0 || type == T_Q8_0) ? 1 : ((type == T_Q4_K || type == T_Q6_K) ? 4 : 8);
  const int gran = 32 / upb > 0 ? 32 / upb : 1;  // blocks that fill all 32 lanes once
  GemvPlan pl;
  int sb = payload_env / ts;
  if (sb >= bpr) sb = bpr;
  else if (sb >= gran) sb = sb / gran * gran;
  if (sb < 1) sb = 1;
  pl.seg_blocks = sb;
  pl.nseg = (bpr + sb - 1) / sb;
  pl.stages = stages_env < 2 ? 2 : stages_env;
  pl.stage_bytes = (int)round_up((int64_t)sb * ts + STAGE_SLACK, 16);
  const int64_t kpad = round_up(K, 512);
  const size_t tables = type == T_IQ2_XXS ? (256 + 128) * 8 : 0;
  const size_t rings = (size_t)GEMV_WARPS * pl.stages * pl.stage_bytes + (size_t)GEMV_WARPS * pl.stages * 8;
  const size_t budget = 110 * 1024;  // at least two CTAs per SM
  int mt = moe ? GEMV_WARPS : 8;
  if (!moe) {
    while (mt > 1 && (mt / 2 >= M || tables + rings + (size_t)mt * (kpad + kpad / 4) > budget)) mt /= 2;
  }
  pl.mt = mt;
  pl.smem = tables + rings + (size_t)mt * (kpad + kpad / 4);
  return pl;
}

template <int TYPE, int MT, typename out_t>
static int launch_cfg(const GemvParams& p, const GemvPlan& pl, int64_t rows, cudaStream_t stream) {
  auto kern = gemv_kernel<TYPE, MT, out_t>;
  if (pl.smem > 227 * 1024) return E_TOO_LARGE;
  static size_t configured[64] = {0};  // per instantiation and device
  int dev = 0;
  cudaGetDevice(&dev);
  if (pl.smem > configured[dev & 63]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem) != cudaSuccess) return E_CUDA;
    configured[dev & 63] = pl.smem;
  }
  const int ctas_per_sm = (MT == 1 && pl.smem <= 74 * 1024) ? 3 : (pl.smem <= 113 * 1024 ? 2 : 1);
  int64_t grid = 148 * ctas_per_sm;
  const int64_t need = (rows + GEMV_WARPS - 1) / GEMV_WARPS;
  if (grid > need) grid = need;
  if (grid < 1) grid = 1;
  return launch_pdl(kern, dim3((unsigned)grid), dim3(GEMV_WARPS * 32), pl.smem, stream, p) == cudaSuccess ? E_OK : E_CUDA;
}

template <int TYPE, typename out_t>
static int launch_mt(GemvParams p, const GemvPlan& pl, int64_t M, cudaStream_t stream) {
  for (int64_t m0 = 0; m0 < M; m0 += pl.mt) {
    p.m0 = (int)m0;
    p.mc = (int)(M - m0 < pl.mt ? M - m0 : pl.mt);
    int rc;
    switch (pl.mt) {
      case 1: rc = launch_cfg<TYPE, 1, out_t>(p, pl, p.n, stream); break;
      case 2: rc = launch_cfg<TYPE, 2, out_t>(p, pl, p.n, stream); break;
      case 4: rc = launch_cfg<TYPE, 4, out_t>(p, pl, p.n, stream); break;
      default: rc = launch_cfg<TYPE, 8, out_t>(p, pl, p.n, stream); break;
    }
    if (rc) return rc;
  }
  return E_OK;
}

template <int TYPE>
static int launch_type(const GemvParams& p, const GemvPlan& pl, int out_dtype, int64_t M, bool moe, cudaStream_t s) {
  if (moe) {
    switch (out_dtype) {
      case DT_F32: return launch_cfg<TYPE, GEMV_WARPS, float>(p, pl, p.n_slots * p.n, s);
      case DT_F16: return launch_cfg<TYPE, GEMV_WARPS, __half>(p, pl, p.n_slots * p.n, s);
      case DT_BF16: return launch_cfg<TYPE, GEMV_WARPS, __nv_bfloat16>(p, pl, p.n_slots * p.n, s);
    }
    return E_BAD_DTYPE;
  }
  switch (out_dtype) {
    case DT_F32: return launch_mt<TYPE, float>(p, pl, M, s);
    case DT_F16: return launch_mt<TYPE, __half>(p, pl, M, s);
    case DT_BF16: return launch_mt<TYPE, __nv_bfloat16>(p, pl, M, s);
  }
  return E_BAD_DTYPE;
}

static int launch_any(GemvParams p, int type, int out_dtype, int64_t M, bool moe, cudaStream_t stream) {
  const GemvPlan pl = make_plan(type, p.k, M, moe);
  p.bpr = (int)(p.k / block_size(type));
  p.seg_blocks = pl.seg_blocks;
  p.nseg = pl.nseg;
  p.stages = pl.stages;
  p.stage_bytes = pl.stage_bytes;
  switch (type) {
    case T_Q4_0: return launch_type<T_Q4_0>(p, pl, out_dtype, M, moe, stream);
    case T_Q8_0: return launch_type<T_Q8_0>(p, pl, out_dtype, M, moe, stream);
    case T_Q4_K: return launch_type<T_Q4_K>(p, pl, out_dtype, M, moe, stream);
    case T_Q6_K: return launch_type<T_Q6_K>(p, pl, out_dtype, M, moe, stream);
    case T_IQ2_XXS: return launch_type<T_IQ2_XXS>(p, pl, out_dtype, M, moe, stream);
    case T_IQ4_XS: return launch_type<T_IQ4_XS>(p, pl, out_dtype, M, moe, stream);
  }
  return E_BAD_TYPE;
}

int launch_gemv(const void* w, const void* xq_soa, void* y, int type, int out_dtype, int64_t M, int64_t N, int64_t K,
                int* status, cudaStream_t stream) {
  if (M == 0 || N == 0) return E_OK;
  static const int use_g1 = gemv_tune_int("GGUF_B200_GEMV1", 1);
  if (M <= 2 && use_g1) {
    const int rc = launch_gemv1(w, xq_soa, y, type, out_dtype, N, K, status, stream, nullptr, (int)M);
    if (rc <= 0) return rc;  // done or failed; 1 = shape outside the register-resident kernel's reach
  }
  // Three or four vectors: two passes of the two-vector register-resident kernel beat the general
  // kernel (14336x4096 Q4_K, 4 vectors: 2 x 9.3 us against 21.7 us), and the types added later exist
  // only in the register-resident kernel, so their larger batches go two vectors at a time as well.
  static const int pair_max = gemv_tune_int("GGUF_B200_GEMV_PAIR_MAX", 4);
  const bool g1_only = type == T_Q4_1 || type == T_Q5_0 || type == T_Q5_1 || type == T_Q5_K || type == T_IQ4_NL || type == T_IQ2_XS ||
                       type == T_IQ2_S || type == T_IQ3_XXS || type == T_IQ3_S || type == T_IQ1_S || type == T_IQ1_M || type == T_Q2_K ||
                       type == T_Q3_K;
  if (g1_only || (use_g1 && M <= pair_max)) {
    bool fell_through = false;
    for (int64_t m0 = 0; m0 < M; m0 += 2) {
      const int rc = launch_gemv1(w, xq_soa, y, type, out_dtype, N, K, status, stream, nullptr, M - m0 >= 2 ? 2 : 1, nullptr, (int)m0, (int)M);
      if (rc == 1 && !g1_only && m0 == 0) {   // shape outside that kernel's reach (decided by the shape alone): the general kernel takes it
        fell_through = true;
        break;
      }
      if (rc) return rc == 1 ? E_TOO_LARGE : rc;   // rows too long for the only kernel these types have
    }
    if (!fell_through) return E_OK;
  }
  GemvParams p{};
  p.w = static_cast<const uint8_t*>(w);
  p.w_bytes = N * (K / block_size(type)) * type_size(type);
  p.xq = static_cast<const uint8_t*>(xq_soa);
  p.m_total = M;
  p.y = y;
  p.n = N;
  p.k = K;
  p.topk_ids = nullptr;
  p.status = status;
  return launch_any(p, type, out_dtype, M, false, stream);
}

int launch_gemv_fused(const void* w, const void* x, void* y, int type, int dtype, int64_t M, int64_t N, int64_t K, int sum_mode,
                      int* status, cudaStream_t stream) {
  // Every CTA quantizes the whole vector for itself, so the saving (one kernel less in the chain
  // before the first dot product) shrinks as K grows and the extra arithmetic grows with it.
  // Measured on B200, per call: K = 1024..4096 one vector 0.5-0.7 us faster (3072x1024 Q8_0 4.5 -> 3.8,
  // 14336x4096 Q4_K 10.7 -> 10.0); K = 8192 even; K = 14336 1.9 us and K = 18944 4.5 us SLOWER, two
  // vectors of K = 4096 1.5 us slower.  Hence: one vector, K up to this bound.
  static const int use = gemv_tune_int("GGUF_B200_GEMV_FUSED_QUANT", 1);
  static const int kmax = gemv_tune_int("GGUF_B200_GEMV_FUSED_QUANT_KMAX", 4096);
  if (!use || M != 1 || K > kmax) return 1;
  return launch_gemv1(w, nullptr, y, type, dtype, N, K, status, stream, nullptr, (int)M, nullptr, 0, 0, x, sum_mode);
}

int launch_moe_gemv(const void* w, const void* xq_soa, void* y, const int32_t* topk_ids, int type, int out_dtype,
                    int64_t tokens, int64_t top_k, int64_t N, int64_t K, int64_t n_experts, int* status,
                    cudaStream_t stream) {
  if (tokens == 0 || N == 0 || top_k == 0) return E_OK;
  static const int use_g1 = gemv_tune_int("GGUF_B200_GEMV1", 1);
  if (use_g1) {   // every (token, expert) pair as a register-resident single-vector GEMV
    GemvMoe moe{topk_ids, tokens, top_k, n_experts, tokens * top_k};
    const int rc = launch_gemv1(w, xq_soa, y, type, out_dtype, N, K, status, stream, nullptr, 1, &moe);
    if (rc <= 0) return rc;
  }
  GemvParams p{};
  p.w = static_cast<const uint8_t*>(w);
  p.w_bytes = n_experts * N * (K / block_size(type)) * type_size(type);
  p.xq = static_cast<const uint8_t*>(xq_soa);
  p.m_total = tokens;
  p.m0 = 0;
  p.mc = 1;
  p.y = y;
  p.n = N;
  p.k = K;
  p.topk_ids = topk_ids;
  p.n_slots = tokens * top_k;
  p.top_k = top_k;
  p.expert_rows = N;
  p.n_experts = n_experts;
  p.status = status;
  return launch_any(p, type, out_dtype, tokens, true, stream);
}

}  // namespace gguf_b200
