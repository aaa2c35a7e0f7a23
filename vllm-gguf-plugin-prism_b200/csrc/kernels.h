// Internal launcher declarations shared by the translation units of libgguf_b200.
// (The public C-ABI is include/gguf_b200.h; nothing here is exported.)
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace gguf_b200 {

// output layouts of the q8_1 quantizer (quantize_q8_1.cu)
enum : int { Q8_MODE_REF = 0, Q8_MODE_SOA = 1, Q8_MODE_F16 = 2 };
// correction column appended to the fp16 activation matrix of the tensor-core kernels
enum : int { CORR_NONE = 0, CORR_Q4_0 = 1, CORR_MIN = 2, CORR_PLUS = 3 };   // B-side column: 8*(d8*sum(q8) - s8), -s8, +s8

// Tensor-parallel input of the SoA quantizer (one vector).  A gathered vector lives on every rank
// as "packets": one 32-bit word {16-bit value, 16-bit tag} per element for f16/bf16 outputs, one
// 64-bit word {f32 value, 32-bit tag} for f32, each written by a single store of the producing
// GEMV (possibly on another GPU).  The quantizer reads x'[k] = x[k] + add_scale * value(add[k])
// (x may be null), polling every packet until its tag equals *add_epoch (bounded by limit_cycles,
// then *status = E_TIMEOUT).  bump != null: thread 0 of the grid increments *bump first -- the
// launch number of the GEMV that follows, which that GEMV uses as the tag of its own packets.
struct Q8Tp {
  const void* add = nullptr;        // packets of the vector to add (element type = the x dtype), or null
  const unsigned* add_epoch = nullptr;
  float add_scale = 0.f;
  int add_parts = 1;                // > 1: the slot holds that many fp32 partial vectors (a row-parallel call's), add_stride
  int64_t add_stride = 0;           //      packets apart; their sum, taken in rank order, is the vector that is added
  unsigned* bump = nullptr;
  long long limit_cycles = 0;
  int* status = nullptr;
};
// M = number of OUTPUT rows.  gather_ids (F16 mode only, may be null): output row r quantizes
// input row gather_ids[r] / gather_div; ids outside [0, gather_limit) give a zero row.
int launch_quantize_q8_1(const void* x, int x_dtype, void* out, int64_t M, int64_t K, int mode, int sum_mode,
                         int64_t ldb, int corr_mode, const int32_t* gather_ids, int64_t gather_div, int64_t gather_limit,
                         cudaStream_t stream, int perm = 0, const Q8Tp* tp = nullptr, int act = 0, int64_t x_ld = 0);
// act (F16 mode): 0 = none; 1 = silu, 2 = gelu: the input rows are [gate | up] of x_ld = 2K values and act(gate) * up is quantized
// leading dimension (elements) of the fp16 activation matrix of the tensor-core kernels
int64_t mmq_ldb(int type, int64_t K);
int mmq_corr_mode(int type);
// value order the tensor-core kernel will expect in the fp16 activation matrix for this problem
int mmq_perm(int type, int64_t N, int64_t K, bool moe, int64_t expert_stride_bytes);

// row_ids != null: row gather -- out row r (K values, K a multiple of 256) = weight row row_ids[r] of weight_rows
int launch_dequantize(const void* w, int type, void* out, int out_dtype, int64_t n_elems, int q4k_contract,
                      cudaStream_t stream, const int64_t* row_ids = nullptr, int64_t K = 0, int64_t weight_rows = 0);

// Fused dequant-GEMV over SoA q8_1 activations (see quantize_q8_1.cu for the layout).
// Y[m, n] for m in [0, M); rows of W are N x (K/QK*TS) bytes, contiguous, 16-byte aligned base.
int launch_gemv(const void* w, const void* xq_soa, void* y, int type, int out_dtype, int64_t M, int64_t N, int64_t K,
                int* status, cudaStream_t stream);
// The whole decode op for M <= 2 vectors in ONE launch (activations quantized inside the GEMV kernel);
// returns 1 when the shape needs the two-kernel route.
int launch_gemv_fused(const void* w, const void* x, void* y, int type, int dtype, int64_t M, int64_t N, int64_t K, int sum_mode,
                      int* status, cudaStream_t stream);
// One- and two-vector specialisation (gemv1.cu): activations in registers.  Returns 1 when the
// shape is outside its reach (the caller then uses the general kernel).
// Tensor-parallel output of the single-vector kernel: every result is sent to all `world` ranks
// as a packet at ll_peer[r] + y_off + row (see Q8Tp), tagged with epoch[slot].
struct GemvTp {
  int world, slot;
  const unsigned* epoch;    // this rank's launch counters (incremented by the quantizer before the launch)
  int64_t y_off;
  void* ll_peer[8];
};
// MoE decode through the same kernel: y row s = weights of expert topk_ids[s] (N x K each, back
// to back) times activation vector s / top_k of the `tokens` quantized ones
struct GemvMoe {
  const int32_t* topk_ids;
  int64_t tokens, top_k, n_experts, slots;
};
int launch_gemv1(const void* w, const void* xq_soa, void* y, int type, int out_dtype, int64_t N, int64_t K, int* status,
                 cudaStream_t stream, const GemvTp* tp = nullptr, int vectors = 1, const GemvMoe* moe = nullptr,
                 int vec0 = 0, int total_vecs = 0,    // vec0 / total_vecs: the `vectors` handled are vec0.. of total_vecs in the scratch
                 const void* x_raw = nullptr, int x_sum_mode = 0);
// x_raw != null (element type = out_dtype): the activations [vectors or tokens][K] are NOT quantized yet and xq_soa is
// ignored -- every CTA quantizes what it needs in shared memory (one launch per GEMV); returns 1 if that does not fit.
// 1 when the q8_1 scratch of this type's GEMV must hold d * sum(q) instead of the fp16 sum of the inputs
inline int gemv_sum_mode(int type) { return (type == 12 || type == 13) ? 1 : 0; }   // Q4_K, Q5_K
// Packets of `nslots` gathered vectors (slot_packets apart) -> plain vectors out[s][0..n) (out_stride
// elements apart); every packet is polled until its tag equals epoch[slot0 + s] (bounded).
// one thread waits (bounded) until flag[slot] has reached world * epoch[slot]
int launch_tp_wait(const unsigned* flag, const unsigned* epoch, int slot, int world, long long limit_cycles, int* status,
                   cudaStream_t stream);
int launch_tp_unpack(const void* packets, const unsigned* epoch, int slot0, int nslots, int64_t slot_packets, int64_t n,
                     void* out, int64_t out_stride, int dtype, long long limit_cycles, int* status, cudaStream_t stream);
int launch_tp_unpack_sum(const void* packets, const unsigned* epoch, int slot, int64_t slot_bytes, int64_t n, int parts, void* out,
                         int dtype, long long limit_cycles, int* status, cudaStream_t stream);
// per-(token,expert) GEMV of the small-batch MoE entry point
int launch_moe_gemv(const void* w, const void* xq_soa, void* y, const int32_t* topk_ids, int type, int out_dtype,
                    int64_t tokens, int64_t top_k, int64_t N, int64_t K, int64_t n_experts, int* status,
                    cudaStream_t stream);

// Tensor-core (tcgen05) dequant-GEMM.  B operand = fp16/bf16 matrix [rows][ldb] (K-major).
// Tensor-parallel output of the tensor-core GEMM: this rank's [M][N] result is column block
// [col_off, col_off + N) of a gathered [M][ld] matrix that every rank holds; the kernel stores its
// tiles into ALL ranks' copies (y_peer[r], plain 16-byte stores over NVLink, this rank included),
// and the last CTA to finish increments epoch[slot] and then flag_peer[r][slot] on every rank.
struct MmqTp {
  int world, slot;
  int64_t col_off, ld;
  unsigned* epoch;
  void* y_peer[8];
  unsigned* flag_peer[8];
};
struct MmqArgs {
  const void* w;            // packed weights (expert 0 for MoE)
  const void* b;            // activation matrix, K-major, element type b_dtype (DT_F16 / DT_BF16)
  void* y;                  // output [rows_out][N], element type out_dtype
  int type, out_dtype, b_dtype;
  int64_t M;                // activation rows (tokens)
  int64_t N, K;             // weight rows, weight columns (values)
  int64_t ldb;              // leading dimension of b in elements
  int64_t kext;             // contraction length in elements incl. correction columns (multiple of 64)
  int corr_mode;            // which correction the appended columns hold
  int perm;                 // value order inside each group of four of b: 0 natural, 1 = (0,2,1,3) (see mmq_perm)
  // MoE gather (null sorted_ids = dense)
  const int32_t* sorted_ids;
  const int32_t* expert_ids;
  const int32_t* n_post_pad;
  int64_t n_sorted, expert_stride_bytes, top_k, rows_out;
  int64_t n_experts;        // experts in w (0: unknown, ids are only limited to [0, 255] as in the reference)
  int moe_block;
  const float* row_scale;   // MoE: output row r is multiplied by row_scale[r] (routing weights); null: no scaling
  int* status;
  const MmqTp* tp;          // null: plain output y
  void* part;               // optional fp32 scratch for split-K partial tiles (16-byte aligned), part_bytes long
  int64_t part_bytes;
};
// bytes of fp32 scratch a dense M x N x K problem can use for split K (0: it never splits)
int64_t mmq_split_scratch_bytes(int64_t M, int64_t N, int64_t K);
int launch_mmq(const MmqArgs& a, cudaStream_t stream);
int mmq_moe_block_size();

int64_t q8_soa_bytes(int64_t M, int64_t K);

// fused MoE step (moe_fused.cu)
int64_t moe_align_sorted_len(int64_t slots, int n_experts, int block);
int launch_moe_align(const int32_t* topk_ids, int64_t slots, int n_experts, int block, int32_t* scratch, int32_t* sorted_ids,
                     int32_t* expert_ids, int32_t* n_post_pad, cudaStream_t stream);
int launch_moe_sum(const void* y, void* out, const int32_t* topk_ids, int n_experts, int64_t tokens, int64_t top_k, int64_t h,
                   int dtype, cudaStream_t stream);

// Device address of the library's one status word on the current device (the word that
// gguf_b200_last_status reads and clears); null if the runtime refuses the lookup.
int* status_word_ptr();

}  // namespace gguf_b200
