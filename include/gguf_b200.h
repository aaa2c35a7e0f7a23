/*
 * gguf_b200 -- C-ABI of the B200 (sm_100a) GGUF quantized-matmul kernels.
 *
 * This is the drop-in boundary: the entry points below are what the reference plugin's
 * native layer (vllm_gguf_plugin/csrc/gguf/gguf_kernel.cu, bound to Python by
 * csrc/torch_bindings.cpp:22-53) does for this path, minus tensor objects.  Plain pointers
 * and sizes only; every function returns 0 or a negative GGUF_B200_E_* code, never throws,
 * never allocates, never synchronises.  Work is enqueued on `stream` (a cudaStream_t passed
 * as void*).  Scratch memory is provided by the caller (gguf_b200_workspace_bytes).
 *
 * Types: GGML ids 2 (Q4_0), 3 (Q4_1), 6 (Q5_0), 7 (Q5_1), 8 (Q8_0), 10 (Q2_K), 11 (Q3_K), 12 (Q4_K), 13 (Q5_K),
 * 14 (Q6_K) -- every type of the reference's tiled kernels -- and 16 (IQ2_XXS), 20 (IQ4_NL), 23 (IQ4_XS); the
 * dequantize and the GEMV entry points (mul_mat_vec_a8, moe_a8_vec and their variants) also take 17 (IQ2_XS),
 * 18 (IQ3_XXS), 19 (IQ1_S), 21 (IQ3_S), 22 (IQ2_S), 29 (IQ1_M) -- all nineteen block types of the reference's dispatch.
 * Weights W are raw GGUF blocks, row-major `uint8 [N][K/QK*type_size]`, base 16-byte aligned.
 * Activations X are `[M][K]` contiguous in `dtype`; outputs Y are `[M][N]` in the same dtype.
 */
#ifndef GGUF_B200_H
#define GGUF_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { GGUF_B200_F32 = 0, GGUF_B200_F16 = 1, GGUF_B200_BF16 = 2 };

enum {
  GGUF_B200_OK = 0,
  GGUF_B200_E_TYPE = -1,      /* block type not supported */
  GGUF_B200_E_DTYPE = -2,     /* dtype not f32/f16/bf16 */
  GGUF_B200_E_SHAPE = -3,     /* K not a multiple of the block size, negative size, ... */
  GGUF_B200_E_POINTER = -4,   /* null or misaligned pointer */
  GGUF_B200_E_WORKSPACE = -5, /* workspace smaller than gguf_b200_workspace_bytes() */
  GGUF_B200_E_CUDA = -6,      /* CUDA runtime error at launch */
  GGUF_B200_E_TOO_LARGE = -7, /* beyond a documented size limit */
  GGUF_B200_E_TIMEOUT = -8    /* a bounded device-side wait expired (reported by gguf_b200_last_status) */
};

enum { GGUF_B200_OP_GEMV = 0, GGUF_B200_OP_MMQ = 1, GGUF_B200_OP_MOE = 2, GGUF_B200_OP_MOE_VEC = 3,
       GGUF_B200_OP_DEQUANT_MATMUL = 4 };

const char* gguf_b200_error_string(int code);
const char* gguf_b200_version(void);

/* bytes per block / values per block of a type, 0 if unsupported
 * (gguf.GGML_QUANT_SIZES; ggml-common.h:17-191) */
int gguf_b200_type_size(int type);
int gguf_b200_block_size(int type);

/* Bytes of one q8_1-quantized activation row: ceil(K/512)*512/32 blocks of 36 bytes
 * (gguf_kernel.cu:114-115: int32 [M][Kpad/32*9]). */
int64_t gguf_b200_q8_1_row_bytes(int64_t K);

/* q8_1 activation quantization, bit-exact with the reference kernel.
 * Replaces: quantize_q8_1 + quantize_row_q8_1_cuda, gguf_kernel.cu:32-85.
 * out: M rows of gguf_b200_q8_1_row_bytes(K) bytes: {half d; half sum; int8 qs[32]} blocks. */
int gguf_b200_quantize_q8_1(const void* x, int dtype, void* out, int64_t M, int64_t K, void* stream);

/* Standalone dequantize, bit-exact with the reference.
 * Replaces: ggml_dequantize, gguf_kernel.cu:87-102 (+ dequantize.cuh:527-571 dispatch).
 * Types: all nineteen (every type of the reference's dispatch).
 * Writes n_elems = m*n values (a multiple of the block size); every output element is
 * written, so the caller need not zero-fill. */
int gguf_b200_dequantize(const void* W, int type, void* out, int out_dtype, int64_t n_elems, void* stream);

/* Embedding look-up: out[r][0..K) = dequantize(weight row row_ids[r]) for r < n_rows, bit-exact with
 * gguf_b200_dequantize of the selected rows.
 * Replaces: index_select of the rows followed by ggml_dequantize in the embedding caller
 * (quantization/vocal_embeds.py:88-96) -- one kernel, no copy of the selected rows.
 * row_ids: int64 on the device; an id outside [0, weight_rows) gives a row of zeros.  K a multiple
 * of 256.  All block types of gguf_b200_dequantize. */
int gguf_b200_dequantize_rows(const void* W, int type, const int64_t* row_ids, int64_t n_rows, int64_t K,
                              int64_t weight_rows, void* out, int out_dtype, void* stream);

/* Scratch bytes an op wants for the given sizes (rows = M, or tokens for the MoE ops).  For the
 * dense GEMM ops this includes room for fp32 partial tiles when the problem is split over K
 * (few output tiles, long rows); a smaller workspace that still holds the activations is
 * accepted and merely disables the split. */
int64_t gguf_b200_workspace_bytes(int op, int type, int64_t M, int64_t N, int64_t K);

/* Decode GEMV: Y[M][N] = q8_1(X) . dequant(W)^T, weights read once for up to 8 vectors.
 * Replaces: ggml_mul_mat_vec_a8, gguf_kernel.cu:104-218 (+ mmvq.cuh). */
int gguf_b200_mul_mat_vec_a8(const void* W, const void* X, void* Y, void* workspace, int64_t workspace_bytes,
                             int type, int dtype, int64_t M, int64_t N, int64_t K, void* stream);

/* The two halves of gguf_b200_mul_mat_vec_a8, for callers that multiply the same activations
 * by several weight matrices (q/k/v, gate/up): quantize once into `workspace`, then run any
 * number of GEMVs on it.
 * Replace: the quantize_row_q8_1_cuda call (gguf_kernel.cu:116-118) and the per-type kernel
 * switch (gguf_kernel.cu:119-215) of ggml_mul_mat_vec_a8 respectively.  `type` matters to the
 * first half only in that Q4_K needs a different sum term than the other types. */
int gguf_b200_gemv_prepare(const void* X, int dtype, void* workspace, int64_t workspace_bytes, int type,
                           int64_t M, int64_t K, void* stream);
int gguf_b200_gemv_prepared(const void* W, const void* workspace, void* Y, int type, int dtype,
                            int64_t M, int64_t N, int64_t K, void* stream);

/* Prefill GEMM on tensor cores (same q8_1-quantized activations).
 * Replaces: ggml_mul_mat_a8, gguf_kernel.cu:220-290 (+ mmq.cuh).  Types 2, 3, 6, 7, 8, 10, 11, 12, 13, 14. */
int gguf_b200_mul_mat_a8(const void* W, const void* X, void* Y, void* workspace, int64_t workspace_bytes,
                         int type, int dtype, int64_t M, int64_t N, int64_t K, void* stream);

/* Fused dequantize + dense GEMM with unquantized activations: Y = X . dequant(W)^T.
 * Replaces the two-step route the reference takes for IQ types at larger batches
 * (quantization/linear.py:50-54: ggml_dequantize then x @ W.T).  dtype f16 or bf16.  Types 16, 20, 23. */
int gguf_b200_dequant_matmul(const void* W, const void* X, void* Y, void* workspace, int64_t workspace_bytes,
                             int type, int dtype, int64_t M, int64_t N, int64_t K, void* stream);

/* MoE expert GEMM over expert-sorted token blocks.
 * Replaces: ggml_moe_a8, gguf_kernel.cu:292-393 (+ moe.cuh:5-129).
 *   X [tokens][K]; W [E][N][K/QK*type_size] with expert_stride_bytes between experts;
 *   sorted_token_ids[n_sorted], expert_ids[ceil(n_sorted/block)], num_tokens_post_padded[1] on device,
 *   as produced by moe_align_block_size with block = gguf_b200_moe_block_size(type);
 *   Y [tokens*top_k][N]: row t = sorted id; rows that receive no token are set to zero.
 *   n_experts (1..256) = experts stored in W: a block whose expert id is outside [0, n_experts) is
 *   skipped, so no id can make the kernel read past W (the reference only guards [0, 255],
 *   moe.cuh:33). */
int gguf_b200_moe_a8(const void* X, const void* W, void* Y, void* workspace, int64_t workspace_bytes,
                     const int32_t* sorted_token_ids, const int32_t* expert_ids,
                     const int32_t* num_tokens_post_padded, int64_t n_sorted, int64_t expert_stride_bytes,
                     int64_t n_experts, int type, int dtype, int64_t tokens, int64_t top_k, int64_t N, int64_t K,
                     void* stream);

/* The whole MoE step of one layer in one call: expert alignment, gate/up expert GEMM, activation,
 * down expert GEMM, routing weights and the sum over the top_k experts.
 * Replaces: the tiled branch of _fused_moe_gguf, quantization/fused_moe.py:56-95 (moe_align_block_size,
 * ggml_moe_a8, apply_moe_activation, ggml_moe_a8, mul_ by the routing weights, moe_sum: six library
 * ops there).  Here the activation runs inside the second GEMM's activation quantizer and the routing
 * weights inside its epilogue; the alignment and the final sum are small kernels of this library.
 *   X [tokens][H]; W13 [E][2I][H/QK*ts] (gate rows, then up rows, of every expert); W2 [E][H][I/QK*ts];
 *   topk_ids int32 [tokens*top_k] and topk_weights float [tokens*top_k] on the device; Y [tokens][H].
 *   act: 1 = silu, 2 = gelu (erf form).  Types 2, 3, 6, 7, 8, 12, 13, 14; n_experts <= 256; I % 8 == 0.
 *   A slot whose expert id is outside [0, n_experts) contributes nothing (expert-parallel masking).
 * Workspace: gguf_b200_fused_moe_workspace_bytes (slot lists, both intermediate matrices, activations). */
int64_t gguf_b200_fused_moe_workspace_bytes(int type13, int type2, int dtype, int64_t tokens, int64_t top_k,
                                            int64_t n_experts, int64_t H, int64_t I);
int gguf_b200_fused_moe(const void* X, const void* W13, const void* W2, void* Y, const int32_t* topk_ids,
                        const float* topk_weights, void* workspace, int64_t workspace_bytes, int type13, int type2,
                        int dtype, int act, int64_t tokens, int64_t top_k, int64_t n_experts, int64_t H, int64_t I,
                        void* stream);

/* Small-batch MoE: one GEMV per (token, expert) pair.
 * Replaces: ggml_moe_a8_vec, gguf_kernel.cu:395-530 (+ moe_vec.cuh:3-53).
 *   topk_ids [tokens*top_k] on device; Y [tokens*top_k][N]. */
int gguf_b200_moe_a8_vec(const void* X, const void* W, void* Y, void* workspace, int64_t workspace_bytes,
                         const int32_t* topk_ids, int64_t n_experts, int type, int dtype, int64_t tokens,
                         int64_t top_k, int64_t N, int64_t K, void* stream);

/* Decode GEMV that needs no workspace from the caller and allocates nothing.  (No counterpart
 * in the reference: its GEMV allocates its scratch tensor inside the call.)
 * For hosts that cannot allocate: an FFI or plain-C integration that only receives W, X and Y
 * from an engine which has already reserved the whole device (weights + KV cache), so that
 * neither a workspace pool nor a late cudaMalloc is available to it.  Same arithmetic and
 * result as gguf_b200_mul_mat_vec_a8; the quantized activations go to a fixed array inside the
 * library (gguf_b200_noalloc_scratch_bytes() = 320 KiB, held by every GPU that loads the
 * library until the process exits).
 * Limits: M <= 8, K <= 32768; beyond them the call returns GGUF_B200_E_TOO_LARGE.
 * The first call on each device resolves the array's device address (one runtime query, made
 * with that device current); make that first call before starting any stream capture.
 * All calls on a device share the one array: calls that may overlap on the GPU (different
 * streams, or another thread) race on it -- serialise them.  Nothing in the array needs to be
 * cleared between calls; each call rewrites all it reads. */
int gguf_b200_mul_mat_vec_a8_noalloc(const void* W, const void* X, void* Y, int type, int dtype,
                                     int64_t M, int64_t N, int64_t K, void* stream);
int64_t gguf_b200_noalloc_scratch_bytes(void);

/* ---- column-sharded tensor parallelism (1..8 GPUs of one NVLink domain) -------------------------
 * No counterpart in the reference: there each rank computes its row shard (the weight loader
 * narrows dim 0, quantization/params.py:227-236) and the serving engine's column-parallel linear
 * layer all-gathers the outputs with a separate NCCL collective.  Here the all-gather is part of
 * the kernels: every rank writes its share of the result straight into ALL ranks' output buffers
 * over NVLink (peer-mapped pointers: symmetric memory or CUDA IPC mappings; plain st.global, no
 * multimem, no TMA).  Rank `rank` of `world` (<= 8) holds rows [rank*N_local, (rank+1)*N_local)
 * of the weight; every rank issues the same sequence of calls.  Calls that can overlap on one GPU
 * must use different slots.  A slot may be reused only after every rank has consumed its previous
 * contents.  Waits on other GPUs are bounded (gguf_b200_set_wait_limit_cycles) and report
 * GGUF_B200_E_TIMEOUT through the status word.
 *
 * Decode, one activation vector.  The gathered vector of call slot `slot` lives on every rank as
 * PACKETS: element i is one naturally aligned word {value, tag} -- 4 bytes {16-bit value, 16-bit
 * tag} for f16/bf16, 8 bytes {f32 value, 32-bit tag} for f32 -- at packet index
 * slot*slot_packets + i of the rank's packet arena (packet_peers[r] = base of rank r's arena,
 * 16-byte aligned, zero before first use; slot_packets >= world*N_local).  tag = number of the
 * launch that wrote it = epochs_local[slot] (uint32 per slot, zero before first use, incremented
 * once per call by this entry point on the device, so captured graphs replay without a reset).
 * A reader that finds the expected tag has the value: no fence, no flag, one NVLink crossing.
 * Activations: x'[k] = X[k] + add_scale * gathered[add_slot][k] rounded to `dtype` (add_slot < 0:
 * x' = X; X may be null when add_slot >= 0) -- the quantizer of this call polls the packets of
 * add_slot itself, so a chain of dependent decode GEMVs needs no collective or wait kernel at all.
 * Returns GGUF_B200_E_TOO_LARGE when the rows are too long for the single-vector kernel.
 * add_parts = 1 when add_slot holds a gathered vector; = world when it holds the fp32 partial
 * vectors of a row-parallel call (below), whose sum is then what is added. */
int gguf_b200_mul_mat_vec_a8_tp(const void* W, const void* X, void* const* packet_peers, uint32_t* epochs_local,
                                int slot, int add_slot, float add_scale, int add_parts, int64_t slot_packets, void* ws,
                                int64_t ws_bytes, int type, int dtype, int64_t N_local, int64_t K, int rank, int world,
                                void* stream);
/* Row-parallel (K-sharded) decode with the all-reduce fused in.  Reference: the loader narrows dim 1
 * of a row-parallel layer's weight to whole blocks (quantization/params.py:238-265) and the serving
 * engine all-reduces the partial outputs with a separate NCCL collective.  Here rank `rank` holds
 * W_local = uint8 [N][K_local/QK*type_size] (its K_local columns of every row) and X_local, its
 * K_local elements of the activation vector; its GEMV sends the fp32 partial sums to ALL ranks as
 * 8-byte packets {f32, tag32} (partial vector r at packet index r*N of the slot, counted in 8-byte
 * packets from the slot's first byte; the slot has slot_packets packet units of 4 bytes for
 * f16/bf16 arenas and 8 for f32 ones, so it needs world*N*8 bytes).  The reduced vector is the sum
 * of the world partial vectors in rank order, rounded once to dtype -- identical bits on every
 * rank -- formed by gguf_b200_tp_unpack_sum or by the activation quantizer of the next tensor-
 * parallel call (add_parts = world).  x'[k] = X_local[k] + add_scale * v[rank*K_local + k] with v
 * the vector in add_slot (gathered: add_parts = 1; reduced: add_parts = world), as above. */
int gguf_b200_mul_mat_vec_a8_tp_rowpar(const void* W_local, const void* X_local, void* const* packet_peers,
                                       uint32_t* epochs_local, int slot, int add_slot, float add_scale, int add_parts,
                                       int64_t slot_packets, void* ws, int64_t ws_bytes, int type, int dtype, int64_t N,
                                       int64_t K_local, int rank, int world, void* stream);
int gguf_b200_tp_unpack_sum(const void* packets_local, const uint32_t* epochs_local, int slot, int64_t slot_packets,
                            int64_t n, int parts, void* out, int dtype, void* stream);
/* Packets -> plain vectors, for consumers that are not one of the calls above: out[s][0..n) =
 * values of slot slot0+s (s < nslots, out rows out_stride elements apart), each packet polled
 * until its tag equals epochs_local[slot0+s]. */
int gguf_b200_tp_unpack(const void* packets_local, const uint32_t* epochs_local, int slot0, int nslots,
                        int64_t slot_packets, int64_t n, void* out, int64_t out_stride, int dtype, void* stream);

/* Prefill, M activation rows: op = GGUF_B200_OP_MMQ (q8_1-quantized activations, types 2/8/12/14)
 * or GGUF_B200_OP_DEQUANT_MATMUL (IQ types, f16/bf16).  y_peers[r] = rank r's gathered output
 * [M][world*N_local] in `dtype` (16-byte aligned; N_local a multiple of 8): the tensor-core kernel's
 * tile epilogue (or, when K is split over CTAs, the kernel that adds the partial tiles) stores this
 * rank's column block [rank*N_local, ...) into every rank's matrix with 16-byte stores.  The last
 * CTA then increments epochs_local[slot] and flag_peers[r][slot] on every rank (uint32 counters,
 * zero before first use, only ever growing).  Workspace: gguf_b200_workspace_bytes(op, type, M,
 * N_local, K). */
int gguf_b200_matmul_tp(int op, const void* W, const void* X, void* const* y_peers, uint32_t* const* flag_peers,
                        uint32_t* epochs_local, int slot, void* ws, int64_t ws_bytes, int type, int dtype, int64_t M,
                        int64_t N_local, int64_t K, int rank, int world, void* stream);
/* Completes the gather of a gguf_b200_matmul_tp call on this rank: a one-thread kernel that waits
 * until flags_local[slot] >= world * epochs_local[slot]; work queued on `stream` behind it may
 * read the full output matrix. */
int gguf_b200_tp_wait(const uint32_t* flags_local, const uint32_t* epochs_local, int slot, int world, void* stream);

/* Limit of every wait on another GPU (packet polls, flag waits), in SM clock cycles; <= 0 restores
 * the default of 2e9 (about a second).  When a wait runs out the kernel stores
 * GGUF_B200_E_TIMEOUT in the status word and returns; the result of that call is invalid. */
void gguf_b200_set_wait_limit_cycles(int64_t cycles);

/* Token-block size the caller must pass to moe_align_block_size.
 * Replaces: ggml_moe_get_block_size, gguf_kernel.cu:532-566 (4 for every type there). */
int gguf_b200_moe_block_size(int type);

/* Device-side status word of the calling thread's current device: 0, or GGUF_B200_E_TIMEOUT if
 * a kernel gave up on a bounded wait since the last call.  Synchronises the device. */
int gguf_b200_last_status(void);

/* Numerics pin (tests only): how Q4_K dequantize combines d*q - m in half precision.
 * 0 = multiply and subtract rounded separately, 1 = one fused multiply-subtract (default:
 * that is what the reference binary does on sm_100a, where the assembler contracts the
 * unqualified mul.f16/sub.f16 pair of dequantize.cuh:193-194). */
void gguf_b200_set_q4k_contract(int fused);

#ifdef __cplusplus
}
#endif
#endif
