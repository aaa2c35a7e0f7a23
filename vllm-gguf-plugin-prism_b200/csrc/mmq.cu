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
// Tile: 128 weight rows (UMMA M) x TN tokens (UMMA N, 32..256) x 64 values per stage.  Operand A
// (the decoded weights) lives in tensor memory: a producer thread owns one weight row = one lane,
// and stores the 64 fp16 values of a stage -- 32 registers -- into 32 columns of that lane with
// tcgen05.st; the MMA takes A from there ([a_tmem] operand form).  Operand B (activations) is
// K-major in shared memory with the 128-byte swizzle, one TMA box per stage.  Weight rows sit on
// the M axis so that small token counts (MoE blocks) do not waste the 128-row instruction.
// Tensor memory: columns [0, TN) the fp32 accumulator, then four or eight A slots of 32 columns.
// Warp roles (P = 4 * groups producer warps, groups = 2 or 4):
//   warps 0..P-1  producers: group g = 128 threads, one per weight row, decodes all 64 values of
//                 its row for the stages i = g, g + groups, ... from the raw-byte ring into the A
//                 slot; afterwards the epilogue (tcgen05.ld, one TMEM lane = one weight row, the
//                 threads of a row split the token columns; tile staged in shared memory and
//                 written by one TMA store, or stored directly for MoE)
//   warp P        B loader: one TMA box of activations per stage; owns the TMEM allocation
//   warp P+1      MMA issuer: warp-uniform loop, an elected lane issues 4 tcgen05.mma + 1 commit per stage
//   warp P+2      raw-weight loader: one 2-D TMA box (256-value chunk x 128 rows) per chunk, or one
//                 padded box per alignment class of rows when rows are not multiples of 16 bytes
// One full/empty mbarrier pair per A slot serves both operands.  K may be split over grid.z
// (fp32 partial tiles, added by add_partials_kernel).  Every wait is bounded in time and
// reports through the status word.
//
// What bounds it (B200, measured on Q4_K 14336 x 4096, 256-token tiles, about 940 clocks per stage
// against 512 of tensor work): no single resource.  Leaving out, one at a time, in builds made for
// the measurement only: the activation loads (every stage reuses the first boxes) -8 %; the decode
// arithmetic (constant operand) -7 %; the tcgen05.mma instructions -23 % (730 clocks per stage
// remain); polling instead of parked barrier waits +2 %.  Neither the number of producer groups
// (2, 4), the depth of the A ring (3, 4) or of the B ring (3, 4), nor the type's decode cost
// (Q8_0 = Q4_K = Q4_0) moves it.  Three stages of 500-730 clocks each -- decode and hand-over
// (about 600 per stage where the other two are small, 64-token tiles), activation boxes (730 with
// the MMAs off, 32 KB per stage and CTA through L2) and the MMAs (512) -- are coupled through the
// shared full / empty barriers of a stage and overlap imperfectly.
#include <cuda.h>

#include <type_traits>

#include "common.cuh"
#include "kernels.h"
#include "mmq_decode.cuh"
#include "tables.cuh"

namespace gguf_b200 {

constexpr int MMQ_ROWS = 128;
constexpr int MMQ_BK = 64;
// Producer groups of 128 threads (one thread per weight row) that take the K stages in turn.
// The whole-stage decoders are short enough for four groups (16 warps) to fit the register
// file; the generic 32-value decoders need more registers per thread and measured faster with
// two groups (IQ2_XXS, the longest decode, and Q2_K, the shortest, gain from four; with four Q6_K
// went 77 -> 92 us, IQ4_XS 80 -> 112 us, Q3_K 88 -> 93 us).  Token tiles of 64 or less
// with a whole-stage decoder run TWO CTAs of two groups per SM instead of one CTA of four: the
// tensor work per stage is small there and the per-stage cost of one MMA-issuing warp is the
// limit, so two independent pipelines per SM raise the rate -- when the grid has enough CTAs to
// put two on every SM (MoE, many row tiles); with fewer CTAs than SMs the one-CTA form keeps
// all 16 decode warps on the tile (`two` is chosen per launch).
__host__ __device__ constexpr int mmq_groups(int type, bool fast, bool two, int tn) {
  return two ? 2 : ((fast || type == T_IQ2_XXS || type == T_Q2_K) ? 4 : 2);
}
__host__ __device__ constexpr int mmq_threads(int type, bool fast, bool two, int tn) { return (4 * mmq_groups(type, fast, two, tn) + 3) * 32; }   // + B loader, MMA issuer, raw-weight loader
// Ring depths.  The decoded weights (operand A) never touch shared memory: a producer thread writes
// the 64 values of its row for one stage -- 32 registers of two fp16 each -- into 32 columns of its own
// lane of tensor memory (tcgen05.st), and the MMA reads its A operand from there.  The A ring is four or
// eight such 32-column slots next to the accumulator's TN columns; it is never shallower than the number
// of producer groups (a group that runs ahead may be at most one use of a slot ahead of the MMA warp,
// or the one-bit phase parity of the slot's barrier would alias).  Eight slots let a group publish its
// next stage while the MMA of its previous one is still queued (Q4_K M = 2048 214 -> 208 us, M = 512
// 62.6 -> 60.1, Q4_0 64.4 -> 61.8); the types that run four groups of 32-value decoders measured slower
// with eight (IQ2_XXS 103 -> 109 us, Q2_K 60 -> 66) and keep four, as do the two-CTA-per-SM kernels, whose
// two allocations must fit the SM's 512 columns.  Shared memory then carries only
// the activations (the B ring, TN * 128 bytes per slot, four slots: the finished tile is staged in
// them, up to TN * 128 fp32 values) and the raw weight bytes.
__host__ __device__ constexpr int mmq_b_stages(int type, bool fast, bool two, int tn) { return 4; }
__host__ __device__ constexpr int mmq_a_stages(int type, bool fast, bool two, int tn) { return (two || type == T_IQ2_XXS || type == T_Q2_K) ? 4 : 8; }
constexpr int MMQ_A_COLS = 32;   // tensor-memory columns of one A slot: 64 fp16 values per lane
__host__ __device__ constexpr uint32_t mmq_tmem_cols(int tn, int a_stages) {
  return (tn < 32 ? 32 : tn) + a_stages * MMQ_A_COLS <= 256 ? 256u : 512u;
}
// per-warp transposition scratch of the types whose correction value is one fp16 of the block (see the producers)
constexpr int MMQ_CORR_ROW = 80;    // bytes per row: 32 fp16 + 16 (an odd number of 16-byte units: conflict-free row reads)
template <int TYPE> __host__ __device__ constexpr int mmq_scratch_bytes(int groups) {
  return Decoder<TYPE, __half>::CORR_OFF >= 0 ? groups * 4 * 32 * MMQ_CORR_ROW : 0;
}
constexpr int MMQ_MAX_RAW = 6;
// shared memory between the operand rings and the raw ring: barriers, then the decoder's tables
__host__ __device__ constexpr int mmq_aux_bytes(int type) { return type == T_IQ2_XXS ? 50176 : 4096; }   // IQ2_XXS: 512 + 16 KB + 32 KB of tables

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
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// one lane of a converged warp (the same one every time)
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
// 32 registers -> 32 consecutive columns of this thread's lane (warp w owns lanes 32 * (w % 4) ...)
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
        "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
        "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// D[tmem] (+)= A[tmem] * B[smem]: A is 128 lanes x 8 columns (16 fp16 values per row, two per column)
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
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
// bounded wait; `code` and `i` name the waiter and its stage for whoever instruments a time-out
__device__ __forceinline__ bool wait_or_note(uint64_t* bar, uint32_t parity, int code, int i) {
  (void)code;
  (void)i;
  return mbar_wait_bounded(bar, parity);
}

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
  int n_experts;          // MoE: expert ids outside [0, n_experts) are skipped
  const float* row_scale; // MoE: routing weight of every output row (null: none)
  int raw_tma;            // 1: raw weight chunks arrive as dense 2-D TMA boxes (wmap); 2: as one padded box per alignment class
                          // of rows (see the loader); 0: as one 1-D bulk copy per row and chunk
  int raw_class_log2;     // raw_tma == 2: log2 of the number of alignment classes
  int raw_stages;         // depth of the raw ring
  int64_t w_row0;         // first row of this matrix in wmap (MoE: added to expert * N)
  int y_tma;              // 1: the output tile leaves through shared memory and one TMA store (ymap)
  int ksplit, sps;        // K slices (grid.z) and main stages per slice; > 1: fp32 partial tiles go to ymap slice z
  // tensor-parallel output (tp_world > 0, dense only): see MmqTp
  int tp_world, tp_slot;
  int64_t tp_col_off, tp_ld;
  unsigned* tp_epoch;
  void* tp_y[8];
  unsigned* tp_flag[8];
};

// CTAs of the tensor-parallel launch in flight per call slot that have stored their tiles
__device__ unsigned g_mmq_tp_done[64];

// End of a tensor-parallel launch, called by every thread of a CTA after its stores to the peers:
// CTA barrier, thread 0 fences system-wide and counts the CTA off; the last CTA of the grid
// increments this rank's launch counter and raises the slot's flag on every rank.  The flags only
// grow (one increment per rank and launch), so replays of a captured graph need no reset.
__device__ __forceinline__ void tp_finish(unsigned* epoch, unsigned* const* flag, int world, int slot, unsigned total_ctas) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    unsigned* done = &g_mmq_tp_done[slot & 63];
    const unsigned prev = atomicAdd(done, 1u);
    if (prev == total_ctas - 1) {
      *done = 0;
      __threadfence_system();
      epoch[slot] += 1;
      __threadfence_system();
      for (int r = 0; r < world; ++r) atomicAdd_system(flag[r] + slot, 1u);
    }
  }
}

template <int TYPE, typename ab_t, typename out_t, int TN, bool MOE, bool FAST, bool TWO>
__global__ void __launch_bounds__(mmq_threads(TYPE, FAST, TWO, TN), TWO ? 2 : 1) mmq_kernel(const __grid_constant__ CUtensorMap bmap, const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap ymap, const MmqParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // carve: the swizzled tiles need 1024-byte alignment
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int B_STAGE = TN * MMQ_BK * 2;
  constexpr int SA = mmq_a_stages(TYPE, FAST, TWO, TN), SB = mmq_b_stages(TYPE, FAST, TWO, TN);
  constexpr int NG = mmq_groups(TYPE, FAST, TWO, TN);
  static_assert(NG <= SA, "a producer group may not lap the A ring");
  constexpr int MMQ_PRODUCER_WARPS = 4 * NG;
  // raw ring geometry: dense TMA boxes, or padded slots that each take one row's bulk copy
  const bool tma = FAST || p.raw_tma == 1;
  const int kc = tma ? TmaGeom<TYPE>::KC_T : RawGeom<TYPE>::KC;
  const int rbc = kc / BlockTraits<TYPE>::QK * BlockTraits<TYPE>::TS;
  const int slot = tma ? rbc : RawGeom<TYPE>::SLOT;
  const int RAW_STAGE = MMQ_ROWS * slot;
  const int SPC = kc / MMQ_BK;                  // MMA stages per chunk (a multiple of NG)
  // Split K: CTA z of p.ksplit works on the stages [i_begin, i_begin + nmain) of the row (a
  // multiple of 8, so chunk boundaries and the stage -> group assignment are unchanged); the
  // last one also takes the correction columns.  Below, i and c count from this CTA's first
  // stage / chunk; i_begin and c_begin are added wherever an address is formed.
  const int i_begin = (int)blockIdx.z * p.sps;
  const int nmain = min(p.nmain - i_begin, p.sps);
  const int ncorr = (int)blockIdx.z == p.ksplit - 1 ? p.ncorr : 0;
  const int c_begin = i_begin / SPC;
  const int nchunks = (nmain + SPC - 1) / SPC;
  uint8_t* sB = smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sB + SB * B_STAGE);
  uint8_t* sScr = sB + SB * B_STAGE + mmq_aux_bytes(TYPE);   // barriers and decoder tables sit in between
  uint8_t* sRaw = sScr + mmq_scratch_bytes<TYPE>(NG);
  // One "full" and one "empty" barrier per A slot (tensor memory) serve both operands of a stage, so the
  // MMA thread polls and commits once per stage: full[i % SA] collects the warps of the group that
  // decoded stage i plus the B loader's expect-tx arrival and bytes; empty[i % SA] is the
  // tcgen05.commit after stage i, which frees A slot i % SA and B slot i % SB alike.
  uint64_t* full_a = bars;                    // [8]
  uint64_t* empty_a = bars + 16;              // [8]
  uint64_t* accum = bars + 32;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 33);
  volatile int* gave_up = reinterpret_cast<volatile int*>(tmem_slot + 1);   // set by any thread whose wait ran out
  // A B ring deeper than the A ring gets "full" barriers of its own (a B box for stage i may be under way
  // while A slot i % SA still serves stage i - SA, so it cannot count on that slot's barrier).
  constexpr bool SPLIT_B = SB > SA;
  uint64_t* full_b = bars + 50;               // [6], used when SPLIT_B
  static_assert(SB <= 6, "room for the B barriers");
  uint64_t* raw_full = bars + 34;             // [MMQ_MAX_RAW]
  uint64_t* raw_empty = bars + 34 + MMQ_MAX_RAW;
  int8_t* s_kv = reinterpret_cast<int8_t*>(bars + 48);                 // 16 bytes
  uint4* s_sgn = reinterpret_cast<uint4*>(bars + 64);                   // IQ2_XXS: 8 copies x 128 x 16 bytes at offset 512
  uint2* s_sel = reinterpret_cast<uint2*>(s_sgn + 8 * 128);             // IQ2_XXS: 16 copies x 256 x 8 bytes

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t n0 = (int64_t)blockIdx.x * MMQ_ROWS;
  const int64_t t0 = (int64_t)blockIdx.y * TN;
  const uint8_t* wbase = p.w;
  if (MOE) {
    const int e = p.expert_ids[blockIdx.y];
    if (e < 0 || e >= p.n_experts) return;           // the reference guards [0, 255] (moe.cuh:33); here also the real expert count
    if (t0 >= (int64_t)p.n_post_pad[0]) return;      // nothing routed to this block
    wbase += (int64_t)e * p.expert_stride_bytes;
  }
  constexpr uint32_t TMEM_COLS = mmq_tmem_cols(TN, SA);
  constexpr uint32_t A_COL0 = TN < 32 ? 32 : TN;   // first column of the A ring, right of the accumulator
  const int nk = nmain + ncorr;

  if (threadIdx.x == 0) {
    for (int s = 0; s < SA; ++s) {
      mbar_init(&full_a[s], MMQ_PRODUCER_WARPS / NG + (SPLIT_B ? 0 : 1));   // the warps of the one group that fills the stage (+ the B loader)
      mbar_init(&empty_a[s], 1);
    }
    if constexpr (SPLIT_B)
      for (int s = 0; s < SB; ++s) mbar_init(&full_b[s], 1);
    mbar_init(accum, 1);
    *gave_up = 0;
    for (int s = 0; s < MMQ_MAX_RAW; ++s) {
      mbar_init(&raw_full[s], 1);
      mbar_init(&raw_empty[s], MMQ_PRODUCER_WARPS);
    }
    fence_barrier_init();
  }
  if (TYPE == T_IQ2_XXS) {
    for (int i = threadIdx.x; i < 16 * 256; i += blockDim.x) s_sel[i] = iq2xxs_pair_selectors(d_iq2xxs_grid[i >> 4]);
    for (int i = threadIdx.x; i < 8 * 128; i += blockDim.x) s_sgn[i] = iq2xxs_pair_signs(d_ksigns_iq2xs[i >> 3]);
  }
  if ((TYPE == T_IQ4_XS || TYPE == T_IQ4_NL) && threadIdx.x < 16) s_kv[threadIdx.x] = d_kvalues_iq4nl[threadIdx.x];
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
    // ---------------- A producers ----------------
    // Thread r of group g decodes all 64 values of row n0 + r for the stages i = g, g + NG, ...:
    // the groups work on different stages at the same time, which hides the latency of one
    // thread's decode chain behind the other group's.
    const int r = threadIdx.x & 127, g = threadIdx.x >> 7;
    const int64_t n = n0 + r;
    const bool live = n < p.N;
    const uint8_t* row = wbase + (live ? n : 0) * p.row_bytes;
    DecodeCtx cx{smem_u32(s_sel) + 8u * (lane & 15), smem_u32(s_sgn) + 16u * (lane & 7), smem_u32(s_kv)};
    const int nunits = (int)((p.K + 31) / 32);   // 32-value units of a row that exist
    int s = g;                 // A slot of this group's next stage and its phase
    uint32_t ph = 0;
    while (s >= SA) { s -= SA; ph ^= 1u; }
    // this thread's lane of tensor memory (warp w reaches lanes 32 * (w % 4) ...: lane = tile row r), column of A slot 0
    const uint32_t a_lane = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + A_COL0;
    auto publish = [&](const uint32_t (&v)[32], int i) -> bool {   // wait for the slot, store the row, signal the MMA warp
      const bool got = wait_or_note(&empty_a[s], ph ^ 1u, 2, i);
      if (!__all_sync(0xffffffffu, got)) return false;    // (the tensor-memory store below is warp-wide)
      tc_fence_after();
      tmem_st32(a_lane + (uint32_t)(s * MMQ_A_COLS), v);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&full_a[s]);
      s += NG;
      while (s >= SA) { s -= SA; ph ^= 1u; }
      return true;
    };
    int rs = 0;                // raw ring slot and phase (TMA staging)
    uint32_t rph = 0;
    // slot of this thread's row inside a raw stage: the row itself, or (class boxes) class r mod P, then r / P
    const int cl2 = p.raw_tma == 2 ? p.raw_class_log2 : 0;
    const int rslot = ((r & ((1 << cl2) - 1)) << (7 - cl2)) | (r >> cl2);
    auto run = [&](auto G) {
      constexpr int GI = decltype(G)::value;
      for (int c = 0; c < nchunks; ++c) {
        if (ok && !wait_or_note(&raw_full[rs], rph, 1, c)) ok = false;
        if constexpr (FAST) {
          const uint8_t* chunk = sRaw + (size_t)rs * RAW_STAGE + (size_t)r * TmaGeom<TYPE>::RBC_T;
          auto stage = [&](auto SCc) {
            constexpr int SC = decltype(SCc)::value;
            const int i = c * 4 + SC;
            if (i < nmain && ok) {
              uint32_t v[32];
              Stage64<TYPE, ab_t>::template decode<SC>(chunk, v);
              ok = publish(v, i);
            }
          };
          stage(std::integral_constant<int, GI>{});
          if constexpr (NG == 2) stage(std::integral_constant<int, GI + 2>{});
        } else {
          // row pointer such that (pointer + byte offset in the row) lands in this thread's slot of chunk c
          const int64_t beg = n * p.row_bytes + (int64_t)(c + c_begin) * rbc;
          const uint8_t* srow = sRaw + (size_t)rs * RAW_STAGE + (size_t)rslot * slot + (tma ? 0 : (beg & 15)) - (int64_t)(c + c_begin) * rbc;
          for (int i = c * SPC + GI; i < (c + 1) * SPC && i < nmain && ok; i += NG) {
            uint32_t v[32];
            constexpr int RW = Decoder<TYPE, ab_t>::RW;
            if constexpr (decoder_pair_load<TYPE>()) {
              // the two 32-value units of a stage read the same words of the block: one load serves both
              const int u = 2 * (i + i_begin);
              uint32_t (&v0)[16] = *reinterpret_cast<uint32_t (*)[16]>(&v[0]);
              uint32_t (&v1)[16] = *reinterpret_cast<uint32_t (*)[16]>(&v[16]);
              if (live && u + 1 < nunits) {
                uint32_t raw[RW];
                Decoder<TYPE, ab_t>::load(srow, u, raw);
                Decoder<TYPE, ab_t>::decode(srow, u, raw, cx, v0);
                Decoder<TYPE, ab_t>::decode(srow, u + 1, raw, cx, v1);
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = 0;
              }
            } else {
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                const int u = 2 * (i + i_begin) + h;
                uint32_t (&vh)[16] = *reinterpret_cast<uint32_t (*)[16]>(&v[16 * h]);
                if (live && u < nunits) {
                  uint32_t raw[RW];
                  Decoder<TYPE, ab_t>::load(srow, u, raw);
                  Decoder<TYPE, ab_t>::decode(srow, u, raw, cx, vh);
                } else {
#pragma unroll
                  for (int j = 0; j < 16; ++j) vh[j] = 0;
                }
              }
            }
            ok = publish(v, i);
          }
        }
        // this warp is done reading the raw chunk: hand the slot back to the loader
        __syncwarp();
        if (lane == 0) mbar_arrive(&raw_empty[rs]);
        if (++rs == p.raw_stages) { rs = 0; rph ^= 1u; }
      }
      // correction columns (Q4_0 / Q4_K ...): a few stages at the end, straight from global memory
      int i0 = nmain;
      while ((i0 % NG) != GI) ++i0;
      if constexpr (Decoder<TYPE, ab_t>::CORR_OFF >= 0) {
        // The correction value of a block is one fp16 of the block itself (d or m).  A thread that
        // collected the 64 values of its own row would issue 64 two-byte loads whose 32 lanes touch
        // 32 different rows; instead the warp walks its 32 rows and each lane takes one block of the
        // row, so a load instruction touches five or six lines.  The values cross to the row's own
        // thread through this warp's scratch in shared memory ([row][32 values], rows 80 bytes apart), half a
        // stage at a time.
        constexpr int TS_ = BlockTraits<TYPE>::TS;
        const int rb = r - lane;   // first tile row of this warp
        uint8_t* scr = sScr + (size_t)warp * (32 * MMQ_CORR_ROW);
        for (int i = i0; i < nk && ok; i += NG) {
          uint32_t v[32];
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            const int64_t g0 = (int64_t)(i - nmain) * 64 + 32 * hh + lane;   // this lane's block
            const bool h0 = g0 * 32 < p.K;
            __syncwarp();   // the row reads of the previous half are done
#pragma unroll 8
            for (int rr = 0; rr < 32; ++rr) {
              const int ri = rb + rr;
              const bool have = n0 + ri < p.N;
              const uint8_t* src = wbase + (n0 + (have ? ri : 0)) * p.row_bytes + g0 * TS_ + Decoder<TYPE, ab_t>::CORR_OFF;
              const unsigned short a = (have && h0) ? __ldg(reinterpret_cast<const unsigned short*>(src)) : (unsigned short)0;
              *reinterpret_cast<unsigned short*>(scr + rr * MMQ_CORR_ROW + 2 * lane) = a;
            }
            __syncwarp();
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
              const uint4 q = lds128s(smem_u32(scr + lane * MMQ_CORR_ROW + 16 * cc));
              v[16 * hh + 4 * cc] = q.x; v[16 * hh + 4 * cc + 1] = q.y; v[16 * hh + 4 * cc + 2] = q.z; v[16 * hh + 4 * cc + 3] = q.w;
            }
          }
          ok = publish(v, i);
        }
      } else {
        for (int i = i0; i < nk && ok; i += NG) {
          uint32_t v[32];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t (&vh)[16] = *reinterpret_cast<uint32_t (*)[16]>(&v[16 * h]);
            if (live) {
              Decoder<TYPE, ab_t>::corr(row, 2 * (i - nmain) + h, p.K, vh);
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j) vh[j] = 0;
            }
          }
          ok = publish(v, i);
        }
      }
    };
    if (g == 0) run(std::integral_constant<int, 0>{});
    else if (g == 1) run(std::integral_constant<int, 1>{});
    else if constexpr (NG == 4) {
      if (g == 2) run(std::integral_constant<int, 2>{});
      else run(std::integral_constant<int, 3>{});
    }
    // ---------------- epilogue: TMEM lane r = weight row n0 + r; the NG threads of a row split the columns ----------------
    if (ok) ok = wait_or_note(accum, 0, 3, 0);
    tc_fence_after();
    out_t* y = static_cast<out_t*>(p.y);
    const uint32_t lane_addr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
    const int64_t npp = MOE ? (int64_t)p.n_post_pad[0] : 0;
    // columns per thread of the NG threads that share a row: a multiple of 16 (one tcgen05.ld), so with a
    // 32-token tile and four groups only the first two groups take part
    constexpr int CH = TN / NG < 16 ? 16 : TN / NG;
    const int cbeg = g * CH, cend = cbeg + CH < TN ? cbeg + CH : TN;
    if (!MOE && p.y_tma) {
      // Stage the tile as [token][128 rows] in the (now idle) operand stages and let one TMA
      // store write it: full lines to global memory, edges clipped by the tensor map.
      out_t* so = reinterpret_cast<out_t*>(smem);
      float* sf = reinterpret_cast<float*>(smem);       // split K: the partial tile stays fp32
      if (ok) {
#pragma unroll 1
        for (int c0 = cbeg; c0 < cend; c0 += 16) {
          uint32_t acc[16];
          tmem_ld16(lane_addr + (uint32_t)c0, acc);
          tmem_ld_wait();
          if (p.ksplit > 1) {
#pragma unroll
            for (int j = 0; j < 16; ++j) sf[(c0 + j) * MMQ_ROWS + r] = __uint_as_float(acc[j]);
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) so[(c0 + j) * MMQ_ROWS + r] = from_float<out_t>(__uint_as_float(acc[j]));
          }
        }
        fence_proxy_async();
      }
      // every producer thread arrives here, also after a time-out, so the barrier cannot hang
      asm volatile("bar.sync 2, %0;" ::"n"(MMQ_PRODUCER_WARPS * 32) : "memory");
      if (p.tp_world > 0 && p.ksplit == 1) {
        // tensor-parallel: the staged tile ([token][128 rows], 16-byte pieces) goes straight into
        // every rank's gathered matrix, column block tp_col_off, with plain vector stores
        constexpr int PIECES = MMQ_ROWS * (int)sizeof(out_t) / 16;      // per token
        const int tokens_here = (int)min((int64_t)TN, p.M - t0);
        const int rows_here = (int)min((int64_t)MMQ_ROWS, p.N - n0);    // (N is a multiple of 8 here)
        const uint4* src = reinterpret_cast<const uint4*>(smem);
        for (int rk = 0; rk < p.tp_world; ++rk) {
          out_t* dst = static_cast<out_t*>(p.tp_y[rk]);
          for (int e = threadIdx.x; e < tokens_here * PIECES; e += MMQ_PRODUCER_WARPS * 32) {
            const int t = e / PIECES, pc = e - t * PIECES;
            if (pc * (16 / (int)sizeof(out_t)) < rows_here)
              *reinterpret_cast<uint4*>(dst + (t0 + t) * p.tp_ld + p.tp_col_off + n0 + pc * (16 / (int)sizeof(out_t))) = src[t * PIECES + pc];
          }
        }
      } else if (threadIdx.x == 0 && ok) {
        asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(&ymap), "r"(smem_u32(so)),
                     "r"((int)n0), "r"((int)t0), "r"((int)blockIdx.z)
                     : "memory");
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
      }
    } else if (ok) {
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
          if (live && orow < p.rows_out) {
            out_t o = from_float<out_t>(__uint_as_float(acc[j]));
            // routing weight applied as the reference applies it: to the stored value, rounded again
            if (MOE && p.row_scale) o = from_float<out_t>(to_float<out_t>(o) * p.row_scale[orow]);
            y[orow * p.N + n] = o;
          }
        }
      }
    }
  } else if (warp == MMQ_PRODUCER_WARPS) {
    // ---------------- B loader: one TMA box (64 k x TN rows) per stage ----------------
    if (lane == 0) {
      // B slot i % SB held stage i - SB: wait for that stage's commit (on its A slot's barrier)
      int sa = 0, sb = 0;             // slots of stage i
      int se = 0;                     // A slot of stage i - SB and the phase of that use
      uint32_t phe = 0;
      for (int i = 0; i < nk; ++i) {
        if (i >= SB) {
          if (!wait_or_note(&empty_a[se], phe, 4, i)) { ok = false; break; }
          if (++se == SA) { se = 0; phe ^= 1u; }
        }
        const int64_t col = i < nmain ? (int64_t)(i + i_begin) * MMQ_BK : p.kpad + (int64_t)(i - nmain) * MMQ_BK;
        uint64_t* fb = SPLIT_B ? &full_b[sb] : &full_a[sa];
        mbar_expect_tx(fb, (uint32_t)B_STAGE);
        tma_load_2d(sB + (size_t)sb * B_STAGE, &bmap, (int)col, (int)t0, fb);
        if (++sa == SA) sa = 0;
        if (++sb == SB) sb = 0;
      }
    }
  } else if (warp == MMQ_PRODUCER_WARPS + 2) {
    // ---------------- raw-weight loader ----------------
    if (tma) {
      // one 2-D TMA box (chunk bytes x 128 rows) per chunk
      if (lane == 0) {
        int64_t wrow = p.w_row0 + n0;
        if (MOE) wrow += (int64_t)p.expert_ids[blockIdx.y] * p.N;
        int st = 0;
        uint32_t sph = 0;
        for (int c = 0; c < nchunks; ++c) {
          if (!wait_or_note(&raw_empty[st], sph ^ 1u, 5, c)) { ok = false; break; }
          mbar_expect_tx(&raw_full[st], (uint32_t)RAW_STAGE);
          tma_load_2d(sRaw + (size_t)st * RAW_STAGE, &wmap, (c + c_begin) * (rbc / 4), (int)wrow, &raw_full[st]);
          if (++st == p.raw_stages) { st = 0; sph ^= 1u; }
        }
      }
    } else if (p.raw_tma == 2) {
      // Rows or chunk starts that are not 16-byte aligned, P = 16 / gcd(16, row bytes) alignment classes:
      // the tensor map views the matrix as rows of P weight rows each (P * row bytes IS a multiple of 16),
      // so weight row P*j + k is the piece at byte k * row_bytes of map row j, and rows of one class k
      // share the remainder of their chunk starts modulo 16.  One box per class and chunk -- 128 / P map
      // rows x one padded slot, from the chunk start rounded down to 16 bytes -- replaces 128 / P bulk
      // copies (the bulk copies cost about 90 clocks each on the SM's copy engine, which bounded every
      // kernel that used them); the decoders index from the remainder, exactly as below.  Bytes beyond the
      // end of a map row are zero-filled by the copy engine and never fetched.
      if (lane == 0) {
        int64_t wrow = p.w_row0 + n0;
        if (MOE) wrow += (int64_t)p.expert_ids[blockIdx.y] * p.N;
        const int cl2 = p.raw_class_log2, rows_per = MMQ_ROWS >> cl2;
        int st = 0;
        uint32_t sph = 0;
        for (int c = 0; c < nchunks; ++c) {
          if (!wait_or_note(&raw_empty[st], sph ^ 1u, 5, c)) { ok = false; break; }
          mbar_expect_tx(&raw_full[st], (uint32_t)RAW_STAGE);
          for (int k = 0; k < (1 << cl2); ++k) {
            const int64_t off = (int64_t)k * p.row_bytes + (int64_t)(c + c_begin) * rbc;
            tma_load_2d(sRaw + (size_t)st * RAW_STAGE + (size_t)k * rows_per * slot, &wmap, (int)((off & ~int64_t(15)) >> 2), (int)(wrow >> cl2),
                        &raw_full[st]);
          }
          if (++st == p.raw_stages) { st = 0; sph ^= 1u; }
        }
      }
    } else {
      // Rows that no tensor map can describe (row bytes not a multiple of 16, or chunk starts that are
      // only 2-byte aligned): one 1-D bulk copy per row and chunk, from the row's chunk address rounded
      // down to 16 bytes into the row's padded slot, so the decoders index from the remainder.  Lane l
      // issues the copies of rows l, l + 32, l + 64, l + 96; all of them complete on the chunk's barrier.
      // Nothing is read past the weight buffer: its last (< 16) bytes are fetched with plain loads.
      const int64_t tile_end = (int64_t)p.N * p.row_bytes;   // bytes of this weight matrix (expert)
      const int64_t safe_end = tile_end & ~int64_t(15);
      int st = 0;
      uint32_t sph = 0;
      for (int c = 0; c < nchunks; ++c) {
        const bool got = wait_or_note(&raw_empty[st], sph ^ 1u, 5, c);
        if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
        uint8_t* stage = sRaw + (size_t)st * RAW_STAGE;
        int64_t a0[4], a1[4];
        uint32_t total = 0;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int rr = lane + 32 * q;
          const int64_t nn = n0 + rr;
          a0[q] = a1[q] = 0;
          if (nn < p.N) {
            const int64_t beg = nn * p.row_bytes + (int64_t)(c + c_begin) * rbc;
            int64_t end = beg + rbc;
            const int64_t row_end = (nn + 1) * p.row_bytes;
            if (end > row_end) end = row_end;
            if (end > beg) {
              a0[q] = beg & ~int64_t(15);
              a1[q] = (end + 15) & ~int64_t(15);
              if (a1[q] > safe_end) {   // the buffer's ragged tail: plain loads, visible through the barrier below
                for (int64_t o = safe_end > a0[q] ? safe_end : a0[q]; o < end; ++o) stage[(size_t)rr * slot + (o - a0[q])] = wbase[o];
                a1[q] = safe_end;
              }
              if (a1[q] > a0[q]) total += (uint32_t)(a1[q] - a0[q]);
              else a1[q] = a0[q];
            }
          }
        }
        if (total) asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&raw_full[st])), "r"(total) : "memory");
        __syncwarp();   // every lane's byte count is registered before any copy can complete and before the arrival
#pragma unroll
        for (int q = 0; q < 4; ++q)
          if (a1[q] > a0[q]) bulk_g2s(stage + (size_t)(lane + 32 * q) * slot, wbase + a0[q], (uint32_t)(a1[q] - a0[q]), &raw_full[st]);
        if (lane == 0) mbar_arrive(&raw_full[st]);
        if (++st == p.raw_stages) { st = 0; sph ^= 1u; }
      }
    }
  } else if (warp == MMQ_PRODUCER_WARPS + 1) {
    // ---------------- MMA issuer ----------------
    // The whole warp walks the loop with uniform control flow (slot counters and descriptors stay
    // warp-uniform values); one elected lane issues the tcgen05 instructions.
    {
      const uint32_t idesc = umma_idesc(MMQ_ROWS, TN, sizeof(ab_t) == 2 && std::is_same<ab_t, __nv_bfloat16>::value ? 1 : 0);
      int sa = 0, sb = 0;
      uint32_t pha = 0, phb = 0;
      const uint64_t bd0 = umma_desc_sw128(smem_u32(sB));
      const uint32_t a_ring = tmem_base + A_COL0;
      for (int i = 0; i < nk; ++i) {
        bool got = wait_or_note(&full_a[sa], pha, 6, i);
        if constexpr (SPLIT_B) got = got && wait_or_note(&full_b[sb], phb, 7, i);
        if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
        tc_fence_after();
        const uint64_t bd = bd0 + (uint64_t)(sb * (B_STAGE >> 4));
        const uint32_t at = a_ring + (uint32_t)(sa * MMQ_A_COLS);
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < MMQ_BK / 16; ++kk)  // 16 values = 8 columns of A, 32 bytes of B = +2 in the descriptor's 16-byte units
            umma_f16_ts(tmem_base, at + 8 * kk, bd + 2 * kk, idesc, (i > 0 || kk > 0) ? 1u : 0u);
          umma_commit(&empty_a[sa]);
        }
        __syncwarp();
        if (++sa == SA) { sa = 0; pha ^= 1u; }
        if (++sb == SB) { sb = 0; phb ^= 1u; }
      }
      // committed in every case: `accum` then completes once every tcgen05.mma this warp issued
      // has finished, which is what the exit path below waits for after a time-out
      if (elect_one()) umma_commit(accum);
      __syncwarp();
    }
  }
  if (!ok) {
    if (lane == 0) atomicExch(p.status, E_TIMEOUT);
    *gave_up = 1;
  }
  tc_fence_before();
  __syncthreads();
  if (*gave_up) {
    // A bounded wait ran out somewhere in this CTA (the result is invalid and the status word says
    // so).  Before the tensor memory is released and the CTA retires, everything it started must
    // have finished: the MMA warp's last commit covers the tensor pipe (bounded wait on `accum`),
    // and the bulk copies still in flight depend on nothing and land within microseconds, so a
    // pause far longer than their latency covers them.  Nothing here can wait for ever.
    if (warp == MMQ_PRODUCER_WARPS + 1) mbar_wait_bounded(accum, 0);
    drain_pause();
    tc_fence_before();
    __syncthreads();
  }
  if (warp == MMQ_PRODUCER_WARPS) tmem_dealloc(tmem_base, TMEM_COLS);
  if (!MOE && p.tp_world > 0 && p.ksplit == 1) tp_finish(p.tp_epoch, p.tp_flag, p.tp_world, p.tp_slot, gridDim.x * gridDim.y);
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
  if (M <= 32) return 32;
  if (M <= 64) return 64;
  if (M <= 128) return 128;
  return 256;
}

// Whether the raw weight bytes of this problem can arrive as 2-D TMA boxes: row bytes a multiple
// of 16 and, for MoE, experts stored back to back with whole 128-row tiles per expert so that a
// box never leaves the caller's buffer.  One decision, shared by the activation quantizer (which
// must know the value order of the stage) and the launch.
static bool raw_tma_ok(int type, int64_t N, int64_t K, bool moe, int64_t expert_stride_bytes) {
  static const char* no_tma = getenv("GGUF_B200_MMQ_NO_RAW_TMA");
  if (no_tma && no_tma[0] == '1') return false;
  if (!(type == T_Q4_0 || type == T_Q8_0 || type == T_Q4_K || type == T_Q5_K || type == T_IQ4_XS)) return false;
  const int64_t row_bytes = K / block_size(type) * type_size(type);
  if (K % 32 != 0 || row_bytes % 16 != 0) return false;
  if (moe && (expert_stride_bytes != N * row_bytes || N % MMQ_ROWS != 0)) return false;
  return true;
}
int mmq_perm(int type, int64_t N, int64_t K, bool moe, int64_t expert_stride_bytes) {
  if (!raw_tma_ok(type, N, K, moe, expert_stride_bytes)) return 0;
  switch (type) {
    case T_Q4_0: return Stage64<T_Q4_0, __half>::PERM;
    case T_Q4_K: return Stage64<T_Q4_K, __half>::PERM;
    case T_Q5_K: return Stage64<T_Q5_K, __half>::PERM;
    case T_Q8_0: return Stage64<T_Q8_0, __half>::PERM;
  }
  return 0;
}

// K slices for a problem of `tiles` output tiles and `nmain` 64-value stages per row: as many (up
// to 16) as keep every slice at least 16 stages long and the grid within one wave of 148 SMs.
static int mmq_pick_split(int tiles, int nmain) {
  static const char* env = getenv("GGUF_B200_MMQ_SPLIT");
  if (env && env[0] == '0') return 1;
  for (int s = 16; s >= 2; --s)
    if ((int64_t)tiles * s <= 148 && nmain / s >= 16) return s;
  return 1;
}
// bytes of fp32 scratch the split may use for an M x N output (0 when it can never split)
int64_t mmq_split_scratch_bytes(int64_t M, int64_t N, int64_t K) {
  const int tn = pick_tn(M);
  const int tiles = (int)(((N + MMQ_ROWS - 1) / MMQ_ROWS) * ((M + tn - 1) / tn));
  const int s = mmq_pick_split(tiles, (int)((K + MMQ_BK - 1) / MMQ_BK));
  return s > 1 ? (int64_t)s * M * N * 4 : 0;
}

// y = sum of the fp32 partial slices, added in slice order (deterministic), rounded once
template <typename out_t>
__global__ void __launch_bounds__(256) add_partials_kernel(const float4* __restrict__ part, out_t* __restrict__ y, int64_t n4, int slices) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
    float4 s = part[i];
    for (int z = 1; z < slices; ++z) {
      const float4 v = part[(int64_t)z * n4 + i];
      s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
    y[4 * i] = from_float<out_t>(s.x);
    y[4 * i + 1] = from_float<out_t>(s.y);
    y[4 * i + 2] = from_float<out_t>(s.z);
    y[4 * i + 3] = from_float<out_t>(s.w);
  }
}

// The same sum, stored into every rank's gathered [M][ld] matrix at column col_off (8 outputs =
// one 16-byte store per rank for 16-bit outputs), followed by the tensor-parallel completion.
template <typename out_t>
__global__ void __launch_bounds__(256) add_partials_tp_kernel(const float4* __restrict__ part, int64_t M, int64_t N, int slices,
                                                              MmqParams p) {
  const int64_t n8 = N / 8, total = M * n8, n4 = M * N / 4;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t m = i / n8, c = (i - m * n8) * 8;
    float v[8];
    const int64_t b = (m * N + c) / 4;
    float4 s0 = part[b], s1 = part[b + 1];
    for (int z = 1; z < slices; ++z) {
      const float4 a0 = part[(int64_t)z * n4 + b], a1 = part[(int64_t)z * n4 + b + 1];
      s0.x += a0.x; s0.y += a0.y; s0.z += a0.z; s0.w += a0.w;
      s1.x += a1.x; s1.y += a1.y; s1.z += a1.z; s1.w += a1.w;
    }
    v[0] = s0.x; v[1] = s0.y; v[2] = s0.z; v[3] = s0.w; v[4] = s1.x; v[5] = s1.y; v[6] = s1.z; v[7] = s1.w;
    if (sizeof(out_t) == 4) {
      for (int rk = 0; rk < p.tp_world; ++rk) {
        float4* d = reinterpret_cast<float4*>(static_cast<float*>(p.tp_y[rk]) + m * p.tp_ld + p.tp_col_off + c);
        d[0] = s0;
        d[1] = s1;
      }
    } else {
      out_t o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = from_float<out_t>(v[j]);
      for (int rk = 0; rk < p.tp_world; ++rk)
        *reinterpret_cast<uint4*>(static_cast<out_t*>(p.tp_y[rk]) + m * p.tp_ld + p.tp_col_off + c) = *reinterpret_cast<const uint4*>(o);
    }
  }
  tp_finish(p.tp_epoch, p.tp_flag, p.tp_world, p.tp_slot, gridDim.x);
}

template <int TYPE, typename ab_t, typename out_t, int TN, bool MOE, bool FAST, bool TWO>
static int launch_kernel(const MmqArgs& a, const MmqParams& p, const CUtensorMap& map, int64_t b_rows, bool raw_tma, cudaStream_t stream) {
  EncodeTiledFn enc = encode_fn();
  MmqParams pp = p;
  CUtensorMap wmap = map;   // placeholder when unused
  if (raw_tma) {
    const int64_t map_rows = MOE ? a.N * pp.n_experts : a.N;   // expert ids are limited to [0, n_experts): a box never leaves the caller's buffer
    const cuuint32_t estr[2] = {1, 1};
    const cuuint64_t wd[2] = {(cuuint64_t)(pp.row_bytes / 4), (cuuint64_t)map_rows};
    const cuuint64_t ws[1] = {(cuuint64_t)pp.row_bytes};
    const cuuint32_t wb[2] = {(cuuint32_t)(TmaGeom<TYPE>::RBC_T / 4), (cuuint32_t)MMQ_ROWS};
    if (enc(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(a.w), wd, ws, wb, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return E_CUDA;
  }
  // alignment-class boxes for everything the dense boxes cannot take (see the loader)
  int class_log2 = -1;
  if (!raw_tma) {
    static const char* no_cls = getenv("GGUF_B200_MMQ_NO_CLASS_TMA");
    int cl = 0;
    while (((pp.row_bytes << cl) & 15) != 0 && cl < 4) ++cl;
    const int64_t map_rows = MOE ? a.N * pp.n_experts : a.N;
    const bool ok = !(no_cls && no_cls[0] == '1') && cl <= 3 && a.N % (1 << cl) == 0 && RawGeom<TYPE>::SLOT <= 1024 &&
                    (!MOE || (a.expert_stride_bytes == a.N * pp.row_bytes && a.N % MMQ_ROWS == 0));
    if (ok) {
      const cuuint32_t estr[2] = {1, 1};
      const cuuint64_t wd[2] = {(cuuint64_t)((pp.row_bytes << cl) / 4), (cuuint64_t)(map_rows >> cl)};
      const cuuint64_t ws[1] = {(cuuint64_t)(pp.row_bytes << cl)};
      const cuuint32_t wb[2] = {(cuuint32_t)(RawGeom<TYPE>::SLOT / 4), (cuuint32_t)(MMQ_ROWS >> cl)};
      if (enc(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(a.w), wd, ws, wb, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return E_CUDA;
      class_log2 = cl;
    }
  }
  const size_t ab_bytes = 1024 + (size_t)mmq_b_stages(TYPE, FAST, TWO, TN) * TN * MMQ_BK * 2 + mmq_aux_bytes(TYPE) +
                          mmq_scratch_bytes<TYPE>(mmq_groups(TYPE, FAST, TWO, TN));
  const size_t raw_stage = (size_t)MMQ_ROWS * (raw_tma ? TmaGeom<TYPE>::RBC_T : RawGeom<TYPE>::SLOT);
  const size_t budget = (TWO ? 113 : 226) * 1024;   // two CTAs share the SM's 228 KB (1 KB each is reserved)
  int rs = (int)((budget - ab_bytes) / raw_stage);
  if (rs > MMQ_MAX_RAW) rs = MMQ_MAX_RAW;
  if (rs < 2) rs = 2;
  pp.raw_tma = raw_tma ? 1 : (class_log2 >= 0 ? 2 : 0);
  pp.raw_class_log2 = class_log2 >= 0 ? class_log2 : 0;
  pp.raw_stages = rs;
  pp.w_row0 = 0;
  const size_t smem = ab_bytes + (size_t)rs * raw_stage;
  if (smem > 227 * 1024) return E_TOO_LARGE;
  // Output tile through shared memory + one TMA store when the rows of y allow a tensor map.
  // Split K (few tiles, long rows): grid.z CTAs per tile each write an fp32 partial tile to slice
  // z of the caller's scratch through the same store; a second kernel adds the slices in order.
  CUtensorMap ymap = map;
  pp.y_tma = 0;
  pp.ksplit = 1;
  pp.sps = pp.nmain;
  static const char* no_ytma = getenv("GGUF_B200_MMQ_NO_Y_TMA");
  if (!MOE && (a.N * sizeof(out_t)) % 16 == 0 && (reinterpret_cast<uintptr_t>(a.y) & 15) == 0 && !(no_ytma && no_ytma[0] == '1')) {
    const int tiles = (int)(((a.N + MMQ_ROWS - 1) / MMQ_ROWS) * ((b_rows + TN - 1) / TN));
    int split = mmq_pick_split(tiles, pp.nmain);
    if (!a.part || a.part_bytes < (int64_t)split * a.M * a.N * 4 || (reinterpret_cast<uintptr_t>(a.part) & 15)) split = 1;
    if (split > 1) {
      pp.sps = ((pp.nmain + split - 1) / split + 7) / 8 * 8;
      pp.ksplit = (pp.nmain + pp.sps - 1) / pp.sps;
    }
    const bool part = pp.ksplit > 1;
    if (a.tp && !part) {
      pp.y_tma = 1;   // tensor-parallel, unsplit: the staged tile is stored to the peers by the CTA itself, no tensor map
    } else {
    const size_t es = part ? 4 : sizeof(out_t);
    const cuuint32_t estr[3] = {1, 1, 1};
    const cuuint64_t yd[3] = {(cuuint64_t)a.N, (cuuint64_t)a.M, (cuuint64_t)pp.ksplit};
    const cuuint64_t ys[2] = {(cuuint64_t)a.N * es, (cuuint64_t)a.N * a.M * es};
    const cuuint32_t yb[3] = {(cuuint32_t)MMQ_ROWS, (cuuint32_t)TN, 1};
    const CUtensorMapDataType ydt = (part || std::is_same<out_t, float>::value) ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                    : (std::is_same<out_t, __nv_bfloat16>::value ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
    if (enc(&ymap, ydt, 3, part ? a.part : a.y, yd, ys, yb, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
            CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS) {
      pp.y_tma = 1;
    } else if (a.tp) {
      return E_CUDA;
    } else {
      pp.ksplit = 1;
      pp.sps = pp.nmain;
    }
    }
  }
  if (a.tp && !pp.y_tma) return E_BAD_SHAPE;
  auto kern = mmq_kernel<TYPE, ab_t, out_t, TN, MOE, FAST, TWO>;
  static size_t configured[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (smem > configured[dev & 63]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return E_CUDA;
    configured[dev & 63] = smem;
  }
  dim3 grid((unsigned)((a.N + MMQ_ROWS - 1) / MMQ_ROWS), (unsigned)((b_rows + TN - 1) / TN), (unsigned)pp.ksplit);
  kern<<<grid, mmq_threads(TYPE, FAST, TWO, TN), smem, stream>>>(map, wmap, ymap, pp);
  if (cudaGetLastError() != cudaSuccess) return E_CUDA;
  if (pp.ksplit > 1 && a.tp) {
    const int64_t n8 = a.M * a.N / 8;
    const int blocks = (int)((n8 + 255) / 256 > 148 * 4 ? 148 * 4 : (n8 + 255) / 256);
    add_partials_tp_kernel<out_t><<<blocks, 256, 0, stream>>>(static_cast<const float4*>(a.part), a.M, a.N, pp.ksplit, pp);
    if (cudaGetLastError() != cudaSuccess) return E_CUDA;
  } else if (pp.ksplit > 1) {
    const int64_t n4 = a.M * a.N / 4;
    const int blocks = (int)((n4 + 255) / 256 > 148 * 8 ? 148 * 8 : (n4 + 255) / 256);
    add_partials_kernel<out_t><<<blocks, 256, 0, stream>>>(static_cast<const float4*>(a.part), static_cast<out_t*>(a.y), n4, pp.ksplit);
    if (cudaGetLastError() != cudaSuccess) return E_CUDA;
  }
  return E_OK;
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
  const bool raw_tma = raw_tma_ok(TYPE, a.N, a.K, MOE, a.expert_stride_bytes);
  if constexpr (Stage64<TYPE, ab_t>::FAST) {
    // the whole-stage decoders need the TMA boxes and the activation order they were quantized in
    if (raw_tma && a.perm == Stage64<TYPE, ab_t>::PERM) {
      if constexpr (TN <= 64) {
        // two small CTAs per SM once the grid can put two on every SM (before any split of K)
        const int64_t ctas = ((a.N + MMQ_ROWS - 1) / MMQ_ROWS) * ((b_rows + TN - 1) / TN);
        if (ctas >= 2 * 148) return launch_kernel<TYPE, ab_t, out_t, TN, MOE, true, true>(a, p, map, b_rows, true, stream);
      }
      return launch_kernel<TYPE, ab_t, out_t, TN, MOE, true, false>(a, p, map, b_rows, true, stream);
    }
  }
  if (a.perm != 0) return E_BAD_SHAPE;
  return launch_kernel<TYPE, ab_t, out_t, TN, MOE, false, false>(a, p, map, b_rows, raw_tma, stream);
}

template <int TYPE, typename ab_t, typename out_t>
static int launch_shape(const MmqArgs& a, const MmqParams& p, cudaStream_t s) {
  if (a.sorted_ids) return launch_tn<TYPE, ab_t, out_t, 64, true>(a, p, a.n_sorted, s);
  switch (pick_tn(a.M)) {
    case 32: return launch_tn<TYPE, ab_t, out_t, 32, false>(a, p, a.M, s);
    case 64: return launch_tn<TYPE, ab_t, out_t, 64, false>(a, p, a.M, s);
    case 128: return launch_tn<TYPE, ab_t, out_t, 128, false>(a, p, a.M, s);
    default: {
      const int rc = launch_tn<TYPE, ab_t, out_t, 256, false>(a, p, a.M, s);
      // (two padded raw chunks of the widest rows do not fit beside three 256-token stages)
      return rc == E_TOO_LARGE ? launch_tn<TYPE, ab_t, out_t, 128, false>(a, p, a.M, s) : rc;
    }
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
  p.row_scale = a.row_scale;
  if (a.tp) {
    // the tile leaves through shared memory, in 16-byte pieces: rows and column offsets must allow it
    if (a.sorted_ids || a.tp->world < 1 || a.tp->world > 8 || a.N % 8 != 0 || a.tp->col_off % 8 != 0 || a.tp->ld % 8 != 0) return E_BAD_SHAPE;
    p.tp_world = a.tp->world;
    p.tp_slot = a.tp->slot;
    p.tp_col_off = a.tp->col_off;
    p.tp_ld = a.tp->ld;
    p.tp_epoch = a.tp->epoch;
    for (int r = 0; r < a.tp->world; ++r) {
      if (!a.tp->y_peer[r] || !a.tp->flag_peer[r] || (reinterpret_cast<uintptr_t>(a.tp->y_peer[r]) & 15)) return E_BAD_POINTER;
      p.tp_y[r] = a.tp->y_peer[r];
      p.tp_flag[r] = a.tp->flag_peer[r];
    }
  }
  p.n_experts = a.n_experts > 0 ? (int)(a.n_experts < 256 ? a.n_experts : 256) : 256;
  const bool bf = a.b_dtype == DT_BF16;
  switch (a.type) {
    case T_Q4_0: return bf ? E_BAD_DTYPE : launch_out<T_Q4_0, __half>(a, p, stream);
    case T_Q8_0: return bf ? E_BAD_DTYPE : launch_out<T_Q8_0, __half>(a, p, stream);
    case T_Q4_K: return bf ? E_BAD_DTYPE : launch_out<T_Q4_K, __half>(a, p, stream);
    case T_Q6_K: return bf ? E_BAD_DTYPE : launch_out<T_Q6_K, __half>(a, p, stream);
    case T_Q4_1: return bf ? E_BAD_DTYPE : launch_out<T_Q4_1, __half>(a, p, stream);
    case T_Q5_0: return bf ? E_BAD_DTYPE : launch_out<T_Q5_0, __half>(a, p, stream);
    case T_Q5_1: return bf ? E_BAD_DTYPE : launch_out<T_Q5_1, __half>(a, p, stream);
    case T_Q5_K: return bf ? E_BAD_DTYPE : launch_out<T_Q5_K, __half>(a, p, stream);
    case T_Q2_K: return bf ? E_BAD_DTYPE : launch_out<T_Q2_K, __half>(a, p, stream);
    case T_Q3_K: return bf ? E_BAD_DTYPE : launch_out<T_Q3_K, __half>(a, p, stream);
    // the dequantize-then-matmul route computes and returns in the activations' own 16-bit type
    case T_IQ2_XXS:
      if (a.out_dtype != a.b_dtype) return E_BAD_DTYPE;
      return bf ? launch_shape<T_IQ2_XXS, __nv_bfloat16, __nv_bfloat16>(a, p, stream) : launch_shape<T_IQ2_XXS, __half, __half>(a, p, stream);
    case T_IQ4_XS:
      if (a.out_dtype != a.b_dtype) return E_BAD_DTYPE;
      return bf ? launch_shape<T_IQ4_XS, __nv_bfloat16, __nv_bfloat16>(a, p, stream) : launch_shape<T_IQ4_XS, __half, __half>(a, p, stream);
    case T_IQ4_NL:
      if (a.out_dtype != a.b_dtype) return E_BAD_DTYPE;
      return bf ? launch_shape<T_IQ4_NL, __nv_bfloat16, __nv_bfloat16>(a, p, stream) : launch_shape<T_IQ4_NL, __half, __half>(a, p, stream);
  }
  return E_BAD_TYPE;
}

}  // namespace gguf_b200
