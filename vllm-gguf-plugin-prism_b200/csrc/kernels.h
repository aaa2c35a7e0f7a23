// Internal launcher declarations shared by the translation units of libgguf_b200.
// (The public C-ABI is include/gguf_b200.h; nothing here is exported.)
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace gguf_b200 {

// output layouts of the q8_1 quantizer (quantize_q8_1.cu)
enum : int { Q8_MODE_REF = 0, Q8_MODE_SOA = 1, Q8_MODE_F16 = 2 };
// correction column appended to the fp16 activation matrix of the tensor-core kernels
enum : int { CORR_NONE = 0, CORR_Q4_0 = 1, CORR_MIN = 2 };

// Optional wait of the SoA quantizer (tensor-parallel consumer): before reading x, wait until
// *flag >= *epoch * world (flag raised by every rank's fused-gather GEMV, epoch counted by this
// rank's own); a time-out sets *status.
struct Q8Wait {
  const unsigned* flag = nullptr;
  const unsigned* epoch = nullptr;
  int world = 0;
  int* status = nullptr;
};
// M = number of OUTPUT rows.  gather_ids (F16 mode only, may be null): output row r quantizes
// input row gather_ids[r] / gather_div; ids outside [0, gather_limit) give a zero row.
int launch_quantize_q8_1(const void* x, int x_dtype, void* out, int64_t M, int64_t K, int mode, int sum_mode,
                         int64_t ldb, int corr_mode, const int32_t* gather_ids, int64_t gather_div, int64_t gather_limit,
                         cudaStream_t stream, int perm = 0, const Q8Wait* wait = nullptr);
// leading dimension (elements) of the fp16 activation matrix of the tensor-core kernels
int64_t mmq_ldb(int type, int64_t K);
int mmq_corr_mode(int type);
// value order the tensor-core kernel will expect in the fp16 activation matrix for this problem
int mmq_perm(int type, int64_t N, int64_t K, bool moe, int64_t expert_stride_bytes);

int launch_dequantize(const void* w, int type, void* out, int out_dtype, int64_t n_elems, int q4k_contract,
                      cudaStream_t stream);

// Fused dequant-GEMV over SoA q8_1 activations (see quantize_q8_1.cu for the layout).
// Y[m, n] for m in [0, M); rows of W are N x (K/QK*TS) bytes, contiguous, 16-byte aligned base.
int launch_gemv(const void* w, const void* xq_soa, void* y, int type, int out_dtype, int64_t M, int64_t N, int64_t K,
                int* status, cudaStream_t stream);
// One- and two-vector specialisation (gemv1.cu): activations in registers.  Returns 1 when the
// shape is outside its reach (the caller then uses the general kernel).
// Tensor-parallel output of the single-vector kernel: results go to y_peer[r] + y_off for every
// rank r (peer-mapped pointers), then flag_peer[r][slot] is incremented once per launch.
struct GemvTp {
  int world, slot, rank;
  unsigned* epoch;          // this rank's launch counters: epoch[slot] is incremented by the last CTA
  int64_t y_off;
  void* y_peer[8];
  unsigned* flag_peer[8];
};
// MoE decode through the same kernel: y row s = weights of expert topk_ids[s] (N x K each, back
// to back) times activation vector s / top_k of the `tokens` quantized ones
struct GemvMoe {
  const int32_t* topk_ids;
  int64_t tokens, top_k, n_experts, slots;
};
int launch_gemv1(const void* w, const void* xq_soa, void* y, int type, int out_dtype, int64_t N, int64_t K, int* status,
                 cudaStream_t stream, const GemvTp* tp = nullptr, int vectors = 1, const GemvMoe* moe = nullptr);
// waits until flag[slot] has reached world * epoch[slot]; sets *status on a time-out
int launch_tp_wait(const unsigned* flag, const unsigned* epoch, int slot, int world, int* status, cudaStream_t stream);
// per-(token,expert) GEMV of the small-batch MoE entry point
int launch_moe_gemv(const void* w, const void* xq_soa, void* y, const int32_t* topk_ids, int type, int out_dtype,
                    int64_t tokens, int64_t top_k, int64_t N, int64_t K, int64_t n_experts, int* status,
                    cudaStream_t stream);

// Tensor-core (tcgen05) dequant-GEMM.  B operand = fp16/bf16 matrix [rows][ldb] (K-major).
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
  int moe_block;
  int* status;
  void* part;               // optional fp32 scratch for split-K partial tiles (16-byte aligned), part_bytes long
  int64_t part_bytes;
};
// bytes of fp32 scratch a dense M x N x K problem can use for split K (0: it never splits)
int64_t mmq_split_scratch_bytes(int64_t M, int64_t N, int64_t K);
int launch_mmq(const MmqArgs& a, cudaStream_t stream);
int mmq_moe_block_size();

int64_t q8_soa_bytes(int64_t M, int64_t K);

}  // namespace gguf_b200
