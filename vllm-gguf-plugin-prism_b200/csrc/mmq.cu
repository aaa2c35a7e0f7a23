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
// Warp roles:  warps 0-7 decode weights into the A stage (two threads per row, 32 values each,
// raw bytes prefetched two stages ahead in registers) and later run the epilogue (tcgen05.ld,
// one TMEM lane = one weight row; the two threads of a row split the token columns); warp 8
// issues the TMA loads of the B tile (tiled 2-D tensor map, no multicast) and owns the TMEM
// allocation; warp 9 lane 0 issues tcgen05.mma and commits stage releases.  A 4-deep mbarrier ring
// decouples them.  Every wait is bounded and reports through the status word.
#include <cuda.h>

#include <type_traits>

#include "common.cuh"
#include "kernels.h"
#include "mmq_decode.cuh"
#include "tables.cuh"

namespace gguf_b200 {

constexpr int MMQ_ROWS = 128;
constexpr int MMQ_BK = 64;
__host__ __device__ constexpr int mmq_stages(int tn) { return tn > 128 ? 3 : 4; }
constexpr int MMQ_PRODUCER_WARPS = 8;   // two threads per weight row of a stage: 32 values each
constexpr int MMQ_THREADS = (MMQ_PRODUCER_WARPS + 3) * 32;   // + B loader, MMA issuer, raw-weight loader
constexpr int MMQ_MAX_RAW = 6;
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
  int debug;   // tuning aid (bit mask): 1 no decode, 2 no A store, 4 no MMA, 8 no B load
  int raw_tma;            // 1: raw weight chunks arrive by 2-D TMA boxes (wmap), 0: by cp.async pieces
  int raw_stages;         // depth of the raw ring
  int64_t w_row0;         // first row of this matrix in wmap (MoE: added to expert * N)
};

template <int TYPE, typename ab_t, typename out_t, int TN, bool MOE>
__global__ void __launch_bounds__(MMQ_THREADS, (TN <= 64 ? 2 : 1)) mmq_kernel(const __grid_constant__ CUtensorMap bmap, const __grid_constant__ CUtensorMap wmap, const MmqParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // carve: the swizzled tiles need 1024-byte alignment
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int B_STAGE = TN * MMQ_BK * 2;
  constexpr int MMQ_STAGES = mmq_stages(TN);
  // raw ring geometry: dense TMA boxes or padded cp.async slots
  const int kc = p.raw_tma ? TmaGeom<TYPE>::KC_T : RawGeom<TYPE>::KC;
  const int rbc = kc / BlockTraits<TYPE>::QK * BlockTraits<TYPE>::TS;
  const int slot = p.raw_tma ? rbc : RawGeom<TYPE>::SLOT;
  const int RAW_STAGE = MMQ_ROWS * slot;
  uint8_t* sA = smem;
  uint8_t* sB = smem + MMQ_STAGES * MMQ_A_STAGE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sB + MMQ_STAGES * B_STAGE);
  uint8_t* sRaw = sB + MMQ_STAGES * B_STAGE + 4096;   // barriers and codebooks take the 4 KB in between
  uint64_t* raw_full = bars + 3 * MMQ_STAGES + 2 + 256 + 16 + 2;   // after tmem slot, grid, signs, levels
  uint64_t* raw_empty = raw_full + MMQ_MAX_RAW;
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
      mbar_init(&full_a[s], MMQ_PRODUCER_WARPS);
      mbar_init(&full_b[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(accum, 1);
    for (int s = 0; s < MMQ_MAX_RAW; ++s) {
      mbar_init(&raw_full[s], 1);
      mbar_init(&raw_empty[s], MMQ_PRODUCER_WARPS);
    }
    fence_barrier_init();
  }
  if (TYPE == T_IQ2_XXS) {
    for (int i = threadIdx.x; i < 256; i += blockDim.x) s_grid[i] = d_iq2xxs_grid[i];
    for (int i = threadIdx.x; i < 128; i += blockDim.x) s_signs[i] = d_ksigns_iq2xs[i];
  }
  if (TYPE == T_IQ4_XS && threadIdx.x < 16) s_kv[threadIdx.x] = d_kvalues_iq4nl[threadIdx.x];
  if (warp == MMQ_PRODUCER_WARPS) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  bool ok = true;

  if (warp < MMQ_PRODUCER_WARPS) {
    // ---------------- A producers: threads r and r+128 decode the two 32-value halves of row n0 + r ----------------
    const int r = threadIdx.x & 127, half = threadIdx.x >> 7;
    const int64_t n = n0 + r;
    const bool live = n < p.N;
    const uint8_t* row = wbase + (live ? n : 0) * p.row_bytes;
    DecodeCtx cx{s_grid, s_signs, s_kv};
    const uint32_t row_off = (uint32_t)((r >> 3) * 1024 + (r & 7) * 128);
    const int nunits = (int)((p.K + 31) / 32);   // 32-value units of a row that exist
    // Raw weight bytes reach shared memory in chunks of KC values per row: warp w copies rows
    // w, w+8, ... of the tile, one coalesced 16-byte cp.async per lane and row (a row's chunk is
    // 66..272 contiguous bytes), one chunk ahead of the decode.  Thread-per-row global loads
    // would touch 32 cache lines per warp instruction and stall on the L1 tag stage instead.
    const int SPC = kc / MMQ_BK;                  // MMA stages per chunk
    const int nchunks = (p.nmain + SPC - 1) / SPC;
    const int64_t tile_end = (int64_t)p.N * p.row_bytes;   // bytes of this weight matrix (expert)
    auto issue_chunk = [&](int c) {
      uint8_t* slot0 = sRaw + (size_t)(c % 2) * RAW_STAGE;
      for (int rr = warp; rr < MMQ_ROWS; rr += MMQ_PRODUCER_WARPS) {
        const int64_t nn = n0 + rr;
        if (nn >= p.N) break;
        const int64_t beg = nn * p.row_bytes + (int64_t)c * rbc;
        int64_t end = beg + rbc;
        const int64_t row_end = (nn + 1) * p.row_bytes;
        if (end > row_end) end = row_end;
        const int64_t a0 = beg & ~int64_t(15);
        const int64_t off = a0 + 16 * (int64_t)lane;
        if (off < end) {
          uint8_t* dst = slot0 + (size_t)rr * slot + 16 * lane;
          if (off + 16 <= tile_end) {
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(wbase + off) : "memory");
          } else {  // last bytes of the buffer: never read past its end
            for (int64_t o = off; o < tile_end; o += 2)
              *reinterpret_cast<uint16_t*>(dst + (o - off)) = *reinterpret_cast<const uint16_t*>(wbase + o);
          }
        }
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    };
    // row pointer such that (pointer + byte offset in the row) lands in this thread's slot of chunk c
    auto row_in_chunk = [&](int c) -> const uint8_t* {
      const int64_t beg = n * p.row_bytes + (int64_t)c * rbc;
      const int st = p.raw_tma ? c % p.raw_stages : c % 2;
      return sRaw + (size_t)st * RAW_STAGE + (size_t)r * slot + (p.raw_tma ? 0 : (beg & 15)) - (int64_t)c * rbc;
    };
    if (!p.raw_tma) issue_chunk(0);
    for (int c = 0; c < nchunks; ++c) {   // runs to the end even after a time-out: all 256 threads must meet at the barrier
      if (p.raw_tma) {
        if (ok) ok = mbar_wait_bounded(&raw_full[c % p.raw_stages], (uint32_t)((c / p.raw_stages) & 1));
      } else {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        asm volatile("bar.sync 1, %0;" ::"n"(MMQ_PRODUCER_WARPS * 32) : "memory");   // chunk c landed for everyone; chunk c-1 fully decoded
        if (c + 1 < nchunks) issue_chunk(c + 1);
      }
      const uint8_t* srow = row_in_chunk(c);
      for (int i = c * SPC; i < (c + 1) * SPC && i < p.nmain && ok; ++i) {
        const int s = i % MMQ_STAGES;
        const uint32_t round = (uint32_t)(i / MMQ_STAGES);
        const int u = 2 * i + half;
        uint32_t v[16];
        if (live && u < nunits && !(p.debug & 1)) {
          constexpr int RW = Decoder<TYPE, ab_t>::RW;
          uint32_t raw[RW];
          Decoder<TYPE, ab_t>::load(srow, u, raw);
          Decoder<TYPE, ab_t>::decode(srow, u, raw, cx, v);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = 0;
        }
        ok = mbar_wait_bounded(&empty[s], (round & 1u) ^ 1u);
        if (!ok) break;
        uint8_t* dst = sA + (size_t)s * MMQ_A_STAGE + row_off;
        if (!(p.debug & 2)) {
#pragma unroll
        for (int cc = 0; cc < 4; ++cc)
          *reinterpret_cast<uint4*>(dst + (((4 * half + cc) ^ (r & 7)) << 4)) = make_uint4(v[4 * cc], v[4 * cc + 1], v[4 * cc + 2], v[4 * cc + 3]);
        fence_proxy_async();
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&full_a[s]);
      }
      if (p.raw_tma) {   // this warp is done reading the raw chunk: hand the slot back to the loader
        __syncwarp();
        if (lane == 0) mbar_arrive(&raw_empty[c % p.raw_stages]);
      }
    }
    // correction columns (Q4_0 / Q4_K): a few stages at the end, straight from global memory
    for (int i = p.nmain; i < nk && ok; ++i) {
      const int s = i % MMQ_STAGES;
      const uint32_t round = (uint32_t)(i / MMQ_STAGES);
      uint32_t v[16];
      if (live) {
        Decoder<TYPE, ab_t>::corr(row, 2 * (i - p.nmain) + half, p.K, v);
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = 0;
      }
      ok = mbar_wait_bounded(&empty[s], (round & 1u) ^ 1u);
      if (!ok) break;
      uint8_t* dst = sA + (size_t)s * MMQ_A_STAGE + row_off;
#pragma unroll
      for (int cc = 0; cc < 4; ++cc)
        *reinterpret_cast<uint4*>(dst + (((4 * half + cc) ^ (r & 7)) << 4)) = make_uint4(v[4 * cc], v[4 * cc + 1], v[4 * cc + 2], v[4 * cc + 3]);
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(&full_a[s]);
    }
    // ---------------- epilogue: TMEM lane r = weight row n0 + r; the two threads of a row split the columns ----------------
    if (ok) ok = mbar_wait_bounded(accum, 0);
    if (ok) {
      tc_fence_after();
      out_t* y = static_cast<out_t*>(p.y);
      const uint32_t lane_addr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
      const int64_t npp = MOE ? (int64_t)p.n_post_pad[0] : 0;
      constexpr int CHALF = TN >= 32 ? TN / 2 : TN;          // columns per thread of a row pair
      const int cbeg = TN >= 32 ? half * CHALF : 0;
      const int cend = TN >= 32 ? cbeg + CHALF : (half == 0 ? TN : 0);
#pragma unroll 1
      for (int c0 = cbeg; c0 < cend; c0 += 16) {
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
  } else if (warp == MMQ_PRODUCER_WARPS) {
    // ---------------- B loader: one TMA box (64 k x TN rows) per stage ----------------
    if (lane == 0) {
      for (int i = 0; i < nk; ++i) {
        const int s = i % MMQ_STAGES;
        const uint32_t round = (uint32_t)(i / MMQ_STAGES);
        if (!mbar_wait_bounded(&empty[s], (round & 1u) ^ 1u)) { ok = false; break; }
        const int64_t col = i < p.nmain ? (int64_t)i * MMQ_BK : p.kpad + (int64_t)(i - p.nmain) * MMQ_BK;
        if (p.debug & 8) { mbar_arrive(&full_b[s]); continue; }
        mbar_expect_tx(&full_b[s], (uint32_t)B_STAGE);
        tma_load_2d(sB + (size_t)s * B_STAGE, &bmap, (int)col, (int)t0, &full_b[s]);
      }
    }
  } else if (warp == MMQ_PRODUCER_WARPS + 2) {
    // ---------------- raw-weight loader: one 2-D TMA box (chunk bytes x 128 rows) per chunk ----------------
    if (lane == 0 && p.raw_tma) {
      const int SPC = kc / MMQ_BK;
      const int nchunks = (p.nmain + SPC - 1) / SPC;
      int64_t wrow = p.w_row0 + n0;
      if (MOE) wrow += (int64_t)p.expert_ids[blockIdx.y] * p.N;
      for (int c = 0; c < nchunks; ++c) {
        const int st = c % p.raw_stages;
        const uint32_t round = (uint32_t)(c / p.raw_stages);
        if (!mbar_wait_bounded(&raw_empty[st], (round & 1u) ^ 1u)) { ok = false; break; }
        mbar_expect_tx(&raw_full[st], (uint32_t)RAW_STAGE);
        tma_load_2d(sRaw + (size_t)st * RAW_STAGE, &wmap, c * (rbc / 4), (int)wrow, &raw_full[st]);
      }
    }
  } else if (warp == MMQ_PRODUCER_WARPS + 1) {
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
        if (!(p.debug & 4))
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
  if (warp == MMQ_PRODUCER_WARPS) tmem_dealloc(tmem_base, TMEM_COLS);
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
  // Raw weight bytes: 2-D TMA boxes when the geometry allows (row bytes a multiple of 16 and, for
  // MoE, experts stored back to back with whole tiles per expert so that a box never leaves the
  // caller's buffer), else cp.async pieces issued by the decode warps.
  MmqParams pp = p;
  CUtensorMap wmap = map;   // placeholder when unused
  static const char* no_tma = getenv("GGUF_B200_MMQ_NO_RAW_TMA");
  bool raw_tma = TmaGeom<TYPE>::OK && a.K % 32 == 0 && pp.row_bytes % 16 == 0 && !(no_tma && no_tma[0] == '1');
  int64_t map_rows = a.N;
  if (MOE) {
    raw_tma = raw_tma && a.expert_stride_bytes == a.N * pp.row_bytes && a.N % MMQ_ROWS == 0;
    map_rows = a.N * 256;   // expert ids are limited to [0, 255]; boxes only touch experts that are routed to
  }
  if (raw_tma) {
    const cuuint64_t wd[2] = {(cuuint64_t)(pp.row_bytes / 4), (cuuint64_t)map_rows};
    const cuuint64_t ws[1] = {(cuuint64_t)pp.row_bytes};
    const cuuint32_t wb[2] = {(cuuint32_t)(TmaGeom<TYPE>::RBC_T / 4), (cuuint32_t)MMQ_ROWS};
    if (enc(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(a.w), wd, ws, wb, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      raw_tma = false;
  }
  const size_t ab_bytes = 1024 + (size_t)mmq_stages(TN) * (MMQ_A_STAGE + TN * MMQ_BK * 2) + 4096;
  const size_t raw_stage = (size_t)MMQ_ROWS * (raw_tma ? TmaGeom<TYPE>::RBC_T : RawGeom<TYPE>::SLOT);
  const size_t budget = (TN <= 64 ? 113 : 226) * 1024;   // two CTAs per SM for small token tiles
  int rs = raw_tma ? (int)((budget - ab_bytes) / raw_stage) : 2;
  if (rs > MMQ_MAX_RAW) rs = MMQ_MAX_RAW;
  if (rs < 2) rs = 2;
  pp.raw_tma = raw_tma ? 1 : 0;
  pp.raw_stages = rs;
  pp.w_row0 = 0;
  const size_t smem = ab_bytes + (size_t)rs * raw_stage;
  if (smem > 227 * 1024) return E_TOO_LARGE;
  auto kern = mmq_kernel<TYPE, ab_t, out_t, TN, MOE>;
  static size_t configured[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (smem > configured[dev & 63]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return E_CUDA;
    configured[dev & 63] = smem;
  }
  dim3 grid((unsigned)((a.N + MMQ_ROWS - 1) / MMQ_ROWS), (unsigned)((b_rows + TN - 1) / TN), 1);
  kern<<<grid, MMQ_THREADS, smem, stream>>>(map, wmap, pp);
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
  static const char* dbg = getenv("GGUF_B200_MMQ_DEBUG");
  p.debug = dbg ? atoi(dbg) : 0;
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
