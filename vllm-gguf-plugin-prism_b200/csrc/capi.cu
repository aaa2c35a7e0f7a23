// extern "C" entry points of libgguf_b200 (declared in include/gguf_b200.h): argument
// validation, workspace carving and dispatch to the kernel launchers.  No allocation, no
// synchronisation (except gguf_b200_last_status), no exceptions.
#include "../../include/gguf_b200.h"

#include "common.cuh"
#include "kernels.h"

using namespace gguf_b200;

namespace gguf_b200 {

// Device-side status word written by kernels whose bounded waits expire.
static __device__ int g_status_word;
static int g_q4k_contract = 1;  // the reference binary fuses the pair (established on B200 against it)
// limit of the waits on other GPUs (packets, flags), in SM clock cycles: about a second by default
static const long long kDefaultWaitLimit = 2000000000ll;
static long long g_wait_limit_cycles = kDefaultWaitLimit;

int* status_word_ptr() {
  static int* ptrs[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  int*& p = ptrs[dev & 63];
  if (!p) {
    void* a = nullptr;
    if (cudaGetSymbolAddress(&a, g_status_word) != cudaSuccess) return nullptr;
    p = static_cast<int*>(a);
  }
  return p;
}

static int* status_ptr() { return status_word_ptr(); }

int mmq_corr_mode(int type) {
  switch (type) {
    case T_Q4_0: return CORR_Q4_0;
    case T_Q4_K: case T_Q5_K: return CORR_MIN;
    case T_Q4_1: case T_Q5_1: return CORR_PLUS;
  }
  return CORR_NONE;
}
int64_t mmq_ldb(int type, int64_t K) {
  const int64_t kpad = round_up(K, 512);
  return mmq_corr_mode(type) == CORR_NONE ? kpad : kpad + round_up(kpad / 32, 64);
}

static bool is_mmq_type(int t) {
  return t == T_Q4_0 || t == T_Q8_0 || t == T_Q4_K || t == T_Q6_K || t == T_Q4_1 || t == T_Q5_0 || t == T_Q5_1 || t == T_Q5_K || t == T_Q2_K ||
         t == T_Q3_K;
}
static bool dtype_ok(int d) { return d == DT_F32 || d == DT_F16 || d == DT_BF16; }
static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

static int check_common(const void* W, const void* X, const void* Y, int type, int dtype, int64_t M, int64_t N, int64_t K) {
  if (!type_size(type)) return E_BAD_TYPE;
  if (!dtype_ok(dtype)) return E_BAD_DTYPE;
  if (M < 0 || N < 0 || K <= 0 || K % block_size(type) != 0) return E_BAD_SHAPE;
  if (K > (int64_t)1 << 24 || N > (int64_t)1 << 31 || M > (int64_t)1 << 31) return E_TOO_LARGE;
  if (M == 0 || N == 0) return E_OK;
  if (!W || !X || !Y || !aligned16(W) || !aligned16(X) || !aligned16(Y)) return E_BAD_POINTER;
  return E_OK;
}

}  // namespace gguf_b200

extern "C" {

const char* gguf_b200_version(void) { return "gguf_b200 0.1 (sm_100a)"; }

const char* gguf_b200_error_string(int code) {
  switch (code) {
    case E_OK: return "ok";
    case E_BAD_TYPE: return "unsupported GGML block type (supported: Q4_0=2, Q4_1=3, Q5_0=6, Q5_1=7, Q8_0=8, Q4_K=12, Q5_K=13, Q6_K=14, Q2_K=10, Q3_K=11, IQ2_XXS=16, IQ2_XS=17, IQ3_XXS=18, IQ1_S=19, IQ4_NL=20, IQ3_S=21, IQ2_S=22, IQ4_XS=23, IQ1_M=29; the tensor-core entry points take fewer)";
    case E_BAD_DTYPE: return "unsupported dtype (expected f32=0, f16=1, bf16=2)";
    case E_BAD_SHAPE: return "bad shape (negative size, or K not a multiple of the block size)";
    case E_BAD_POINTER: return "null or misaligned pointer (16-byte alignment required)";
    case E_WORKSPACE: return "workspace too small (see gguf_b200_workspace_bytes)";
    case E_CUDA: return "CUDA runtime error at launch";
    case E_TOO_LARGE: return "size beyond the supported limit";
    case E_TIMEOUT: return "a bounded device-side wait expired";
  }
  return "unknown error";
}

int gguf_b200_type_size(int type) { return dequant_type_size(type); }
int gguf_b200_block_size(int type) { return dequant_block_size(type); }
int64_t gguf_b200_q8_1_row_bytes(int64_t K) { return round_up(K, 512) / 32 * 36; }
void gguf_b200_set_q4k_contract(int fused) { g_q4k_contract = fused ? 1 : 0; }
int gguf_b200_moe_block_size(int type) { return is_mmq_type(type) ? mmq_moe_block_size() : 0; }

void gguf_b200_set_wait_limit_cycles(int64_t cycles) { g_wait_limit_cycles = cycles > 0 ? cycles : kDefaultWaitLimit; }

int gguf_b200_last_status(void) {
  int* p = status_ptr();
  if (!p) return E_CUDA;
  int v = 0;
  if (cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return E_CUDA;
  if (v != 0) {
    int zero = 0;
    cudaMemcpy(p, &zero, sizeof(int), cudaMemcpyHostToDevice);
  }
  return v;
}

int gguf_b200_quantize_q8_1(const void* x, int dtype, void* out, int64_t M, int64_t K, void* stream) {
  if (!dtype_ok(dtype)) return E_BAD_DTYPE;
  if (M < 0 || K <= 0) return E_BAD_SHAPE;
  if (M == 0) return E_OK;
  if (!x || !out || (reinterpret_cast<uintptr_t>(out) & 3)) return E_BAD_POINTER;
  return launch_quantize_q8_1(x, dtype, out, M, K, Q8_MODE_REF, 0, 0, CORR_NONE, nullptr, 1, 0, static_cast<cudaStream_t>(stream));
}

int gguf_b200_dequantize(const void* W, int type, void* out, int out_dtype, int64_t n_elems, void* stream) {
  if (!dequant_type_size(type)) return E_BAD_TYPE;
  if (!dtype_ok(out_dtype)) return E_BAD_DTYPE;
  if (n_elems < 0 || n_elems % dequant_block_size(type) != 0) return E_BAD_SHAPE;
  if (n_elems == 0) return E_OK;
  if (!W || !out || !aligned16(out) || (reinterpret_cast<uintptr_t>(W) & 15)) return E_BAD_POINTER;
  return launch_dequantize(W, type, out, out_dtype, n_elems, g_q4k_contract, static_cast<cudaStream_t>(stream));
}

int gguf_b200_dequantize_rows(const void* W, int type, const int64_t* row_ids, int64_t n_rows, int64_t K,
                              int64_t weight_rows, void* out, int out_dtype, void* stream) {
  if (!dequant_type_size(type)) return E_BAD_TYPE;
  if (!dtype_ok(out_dtype)) return E_BAD_DTYPE;
  if (n_rows < 0 || weight_rows < 0 || K <= 0 || K % 256 != 0) return E_BAD_SHAPE;
  if (n_rows == 0) return E_OK;
  if (!W || !out || !row_ids || !aligned16(out) || !aligned16(W) || (reinterpret_cast<uintptr_t>(row_ids) & 7)) return E_BAD_POINTER;
  return launch_dequantize(W, type, out, out_dtype, n_rows * K, g_q4k_contract, static_cast<cudaStream_t>(stream), row_ids, K, weight_rows);
}

// Up to this many tokens the op is bound by reading the weights once, which the GEMV kernel does
// best; it then runs with the tiled kernels' formulas (Q4_K min term from the stored fp16 sum).
// Measured cross-over on 14336x4096: the types with whole-stage tensor-core decoders win from 5
// tokens on (Q4_K, 8 tokens: 26.9 us against 37.3 us through the GEMV); the others keep the GEMV
// up to 16.
// Largest batch that ggml_mul_mat_a8 serves with the GEMV kernels (tiled formulas) instead of the tensor cores.  Types
// that exist only in the two-vector register-resident GEMV would need a pass per pair of tokens: beyond two passes the
// tiled kernel (about 25 us on a 14336x4096 matrix whatever the batch) is faster.  Q6_K has the multi-vector kernel.
static int64_t mmq_gemv_max_tokens(int type) { return type == T_Q6_K ? 16 : 4; }

// activation matrix of the tensor-core kernels, rounded so that what follows it stays aligned
static int64_t mmq_b_bytes(int type, int64_t M, int64_t K) { return round_up(M * mmq_ldb(type, K) * 2, 256); }

int64_t gguf_b200_workspace_bytes(int op, int type, int64_t M, int64_t N, int64_t K) {
  if (!type_size(type) || M < 0 || K <= 0) return 0;
  switch (op) {
    case GGUF_B200_OP_GEMV:
    case GGUF_B200_OP_MOE_VEC: return q8_soa_bytes(M, K);
    /* dense GEMM: + room for the fp32 partial tiles of a split over K (small N, long K) */
    case GGUF_B200_OP_MMQ: return M <= mmq_gemv_max_tokens(type) ? M * mmq_ldb(type, K) * 2 : mmq_b_bytes(type, M, K) + mmq_split_scratch_bytes(M, N > 0 ? N : 0, K);
    case GGUF_B200_OP_MOE: return M * mmq_ldb(type, K) * 2;  /* M = length of sorted_token_ids */
    case GGUF_B200_OP_DEQUANT_MATMUL: return mmq_split_scratch_bytes(M, N > 0 ? N : 0, K);
  }
  return 0;
}

int gguf_b200_mul_mat_vec_a8(const void* W, const void* X, void* Y, void* ws, int64_t ws_bytes, int type, int dtype,
                             int64_t M, int64_t N, int64_t K, void* stream) {
  int rc = check_common(W, X, Y, type, dtype, M, N, K);
  if (rc || M == 0 || N == 0) return rc;
  if (!ws || !aligned16(ws)) return E_BAD_POINTER;
  if (ws_bytes < q8_soa_bytes(M, K)) return E_WORKSPACE;
  int* st = status_ptr();
  if (!st) return E_CUDA;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // one or two vectors: ONE launch, the GEMV kernel quantizes the activations itself (same codes)
  rc = launch_gemv_fused(W, X, Y, type, dtype, M, N, K, gemv_sum_mode(type), st, s);
  if (rc <= 0) return rc;
  // the Q4_K / Q5_K GEMV takes its min term from the quantized codes (sum_mode 1), all others from the fp16 sum
  rc = launch_quantize_q8_1(X, dtype, ws, M, K, Q8_MODE_SOA, gemv_sum_mode(type), 0, CORR_NONE, nullptr, 1, 0, s);
  if (rc) return rc;
  return launch_gemv(W, ws, Y, type, dtype, M, N, K, st, s);
}

// the activation quantizer's view of the slot whose contents are added to x (both tensor-parallel decode calls)
// (the vector in add_slot has `full` elements; the caller needs those from `first` on)
static int tp_add_setup(Q8Tp& qt, const void* arena_local, const uint32_t* epochs_local, int add_slot, float add_scale, int add_parts,
                        int64_t slot_packets, int64_t psz, int64_t full, int64_t first, int world) {
  if (add_slot < 0) return E_OK;
  if (add_parts != 1 && add_parts != world) return E_BAD_SHAPE;
  if (add_parts == 1 ? full > slot_packets : (int64_t)add_parts * full * 8 > slot_packets * psz) return E_BAD_SHAPE;
  qt.add = static_cast<const uint8_t*>(arena_local) + (int64_t)add_slot * slot_packets * psz + first * (add_parts == 1 ? psz : 8);
  qt.add_epoch = epochs_local + add_slot;
  qt.add_scale = add_scale;
  qt.add_parts = add_parts;
  qt.add_stride = full;
  return E_OK;
}

int gguf_b200_mul_mat_vec_a8_tp(const void* W, const void* X, void* const* packet_peers, uint32_t* epochs_local, int slot,
                                int add_slot, float add_scale, int add_parts, int64_t slot_packets, void* ws, int64_t ws_bytes,
                                int type, int dtype, int64_t N_local, int64_t K, int rank, int world, void* stream) {
  if (!packet_peers || !epochs_local) return E_BAD_POINTER;
  if (world < 1 || world > 8 || rank < 0 || rank >= world || slot < 0 || slot_packets <= 0) return E_BAD_SHAPE;
  if (!X && add_slot < 0) return E_BAD_POINTER;
  int rc = check_common(W, X ? X : W, packet_peers[rank], type, dtype, 1, N_local, K);
  if (rc || N_local == 0) return rc;
  if ((int64_t)world * N_local > slot_packets || add_slot == slot) return E_BAD_SHAPE;
  if (add_slot >= 0 && add_parts != 1 && add_parts != world) return E_BAD_SHAPE;
  if (!ws || !aligned16(ws)) return E_BAD_POINTER;
  if (ws_bytes < q8_soa_bytes(1, K)) return E_WORKSPACE;
  int* st = status_ptr();
  if (!st) return E_CUDA;
  const int64_t psz = dtype == DT_F32 ? 8 : 4;   // bytes per packet
  GemvTp tp{};
  tp.world = world;
  tp.slot = slot;
  tp.epoch = epochs_local;
  tp.y_off = (int64_t)rank * N_local;
  for (int r = 0; r < world; ++r) {
    if (!packet_peers[r] || (reinterpret_cast<uintptr_t>(packet_peers[r]) & 15)) return E_BAD_POINTER;
    tp.ll_peer[r] = static_cast<uint8_t*>(packet_peers[r]) + (int64_t)slot * slot_packets * psz;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  Q8Tp qt{};
  qt.bump = epochs_local + slot;    // this launch's number, read by the GEMV kernel behind the quantizer
  qt.status = st;
  qt.limit_cycles = g_wait_limit_cycles;
  // x' = x + add_scale * (vector gathered, or partial vectors reduced, in add_slot): the quantizer polls its packets
  rc = tp_add_setup(qt, packet_peers[rank], epochs_local, add_slot, add_scale, add_parts, slot_packets, psz, K, 0, world);
  if (rc) return rc;
  rc = launch_quantize_q8_1(X, dtype, ws, 1, K, Q8_MODE_SOA, gemv_sum_mode(type), 0, CORR_NONE, nullptr, 1, 0, s, 0, &qt);
  if (rc) return rc;
  rc = launch_gemv1(W, ws, nullptr, type, dtype, N_local, K, st, s, &tp);
  return rc == 1 ? E_TOO_LARGE : rc;   // rows too long for the single-vector kernel
}

int gguf_b200_mul_mat_vec_a8_tp_rowpar(const void* W_local, const void* X_local, void* const* packet_peers, uint32_t* epochs_local,
                                       int slot, int add_slot, float add_scale, int add_parts, int64_t slot_packets, void* ws,
                                       int64_t ws_bytes, int type, int dtype, int64_t N, int64_t K_local, int rank, int world,
                                       void* stream) {
  if (!packet_peers || !epochs_local) return E_BAD_POINTER;
  if (world < 1 || world > 8 || rank < 0 || rank >= world || slot < 0 || slot_packets <= 0) return E_BAD_SHAPE;
  if (!X_local && add_slot < 0) return E_BAD_POINTER;
  int rc = check_common(W_local, X_local ? X_local : W_local, packet_peers[rank], type, dtype, 1, N, K_local);
  if (rc || N == 0) return rc;
  const int64_t psz = dtype == DT_F32 ? 8 : 4;   // bytes per packet unit of the arena (the partials always take 8)
  if ((int64_t)world * N * 8 > slot_packets * psz || add_slot == slot) return E_BAD_SHAPE;
  if (add_slot >= 0 && add_parts != 1 && add_parts != world) return E_BAD_SHAPE;
  if (!ws || !aligned16(ws)) return E_BAD_POINTER;
  if (ws_bytes < q8_soa_bytes(1, K_local)) return E_WORKSPACE;
  int* st = status_ptr();
  if (!st) return E_CUDA;
  GemvTp tp{};
  tp.world = world;
  tp.slot = slot;
  tp.epoch = epochs_local;
  tp.y_off = (int64_t)rank * N;    // partial vector r sits N fp32 packets after partial vector r - 1
  for (int r = 0; r < world; ++r) {
    if (!packet_peers[r] || (reinterpret_cast<uintptr_t>(packet_peers[r]) & 15)) return E_BAD_POINTER;
    tp.ll_peer[r] = static_cast<uint8_t*>(packet_peers[r]) + (int64_t)slot * slot_packets * psz;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  Q8Tp qt{};
  qt.bump = epochs_local + slot;
  qt.status = st;
  qt.limit_cycles = g_wait_limit_cycles;
  // (this rank's slice of the vector in add_slot: gathered or reduced vectors are indexed from the slice's first element)
  rc = tp_add_setup(qt, packet_peers[rank], epochs_local, add_slot, add_scale, add_parts, slot_packets, psz, (int64_t)world * K_local,
                    (int64_t)rank * K_local, world);
  if (rc) return rc;
  rc = launch_quantize_q8_1(X_local, dtype, ws, 1, K_local, Q8_MODE_SOA, gemv_sum_mode(type), 0, CORR_NONE, nullptr, 1, 0, s, 0, &qt);
  if (rc) return rc;
  rc = launch_gemv1(W_local, ws, nullptr, type, DT_F32, N, K_local, st, s, &tp);   // fp32 partial sums travel as 8-byte packets
  return rc == 1 ? E_TOO_LARGE : rc;
}

int gguf_b200_tp_unpack_sum(const void* packets_local, const uint32_t* epochs_local, int slot, int64_t slot_packets, int64_t n,
                            int parts, void* out, int dtype, void* stream) {
  if (!packets_local || !epochs_local || !out) return E_BAD_POINTER;
  if (!dtype_ok(dtype)) return E_BAD_DTYPE;
  const int64_t psz = dtype == DT_F32 ? 8 : 4;
  if (slot < 0 || n < 0 || parts < 1 || parts > 8 || (int64_t)parts * n * 8 > slot_packets * psz) return E_BAD_SHAPE;
  int* st = status_ptr();
  if (!st) return E_CUDA;
  return launch_tp_unpack_sum(packets_local, epochs_local, slot, slot_packets * psz, n, parts, out, dtype, g_wait_limit_cycles, st,
                              static_cast<cudaStream_t>(stream));
}

int gguf_b200_tp_unpack(const void* packets_local, const uint32_t* epochs_local, int slot0, int nslots, int64_t slot_packets,
                        int64_t n, void* out, int64_t out_stride, int dtype, void* stream) {
  if (!packets_local || !epochs_local || !out) return E_BAD_POINTER;
  if (!dtype_ok(dtype)) return E_BAD_DTYPE;
  if (slot0 < 0 || nslots < 0 || n < 0 || n > slot_packets || out_stride < n) return E_BAD_SHAPE;
  int* st = status_ptr();
  if (!st) return E_CUDA;
  return launch_tp_unpack(packets_local, epochs_local, slot0, nslots, slot_packets, n, out, out_stride, dtype, g_wait_limit_cycles,
                          st, static_cast<cudaStream_t>(stream));
}

int gguf_b200_matmul_tp(int op, const void* W, const void* X, void* const* y_peers, uint32_t* const* flag_peers,
                        uint32_t* epochs_local, int slot, void* ws, int64_t ws_bytes, int type, int dtype, int64_t M,
                        int64_t N_local, int64_t K, int rank, int world, void* stream) {
  if (!y_peers || !flag_peers || !epochs_local) return E_BAD_POINTER;
  if (world < 1 || world > 8 || rank < 0 || rank >= world || slot < 0) return E_BAD_SHAPE;
  if (op != GGUF_B200_OP_MMQ && op != GGUF_B200_OP_DEQUANT_MATMUL) return E_BAD_SHAPE;
  int rc = check_common(W, X, y_peers[rank], type, dtype, M, N_local, K);
  if (rc || M == 0 || N_local == 0) return rc;
  if (op == GGUF_B200_OP_DEQUANT_MATMUL) {
    if (type != T_IQ2_XXS && type != T_IQ4_XS && type != T_IQ4_NL) return E_BAD_TYPE;
    if (dtype != DT_F16 && dtype != DT_BF16) return E_BAD_DTYPE;
    if (K % 64 != 0) return E_BAD_SHAPE;
  } else if (!is_mmq_type(type)) {
    return E_BAD_TYPE;
  }
  int* st = status_ptr();
  if (!st) return E_CUDA;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  MmqTp tp{};
  tp.world = world;
  tp.slot = slot;
  tp.col_off = (int64_t)rank * N_local;
  tp.ld = (int64_t)world * N_local;
  tp.epoch = epochs_local;
  for (int r = 0; r < world; ++r) {
    tp.y_peer[r] = y_peers[r];
    tp.flag_peer[r] = flag_peers[r];
  }
  MmqArgs a{};
  a.w = W; a.y = nullptr;
  a.type = type; a.out_dtype = dtype;
  a.M = M; a.N = N_local; a.K = K;
  a.rows_out = M;
  a.status = st;
  a.tp = &tp;
  if (op == GGUF_B200_OP_DEQUANT_MATMUL) {
    a.b = X; a.b_dtype = dtype; a.ldb = K;
    a.corr_mode = CORR_NONE;
    if (ws && aligned16(ws) && ws_bytes > 0) {
      a.part = ws;
      a.part_bytes = ws_bytes;
    }
    return launch_mmq(a, s);
  }
  if (!ws || !aligned16(ws)) return E_BAD_POINTER;
  const int64_t ldb = mmq_ldb(type, K);
  if (ws_bytes < M * ldb * 2) return E_WORKSPACE;
  const int perm = mmq_perm(type, N_local, K, false, 0);
  rc = launch_quantize_q8_1(X, dtype, ws, M, K, Q8_MODE_F16, 0, ldb, mmq_corr_mode(type), nullptr, 1, 0, s, perm);
  if (rc) return rc;
  a.perm = perm;
  a.b = ws; a.b_dtype = DT_F16; a.ldb = ldb;
  a.corr_mode = mmq_corr_mode(type);
  const int64_t used = mmq_b_bytes(type, M, K);
  if (ws_bytes > used) {
    a.part = static_cast<uint8_t*>(ws) + used;
    a.part_bytes = ws_bytes - used;
  }
  return launch_mmq(a, s);
}

int gguf_b200_tp_wait(const uint32_t* flags_local, const uint32_t* epochs_local, int slot, int world, void* stream) {
  if (!flags_local || !epochs_local) return E_BAD_POINTER;
  if (world < 1 || world > 8 || slot < 0) return E_BAD_SHAPE;
  int* st = status_ptr();
  if (!st) return E_CUDA;
  return launch_tp_wait(flags_local, epochs_local, slot, world, g_wait_limit_cycles, st, static_cast<cudaStream_t>(stream));
}

int gguf_b200_gemv_prepare(const void* X, int dtype, void* ws, int64_t ws_bytes, int type, int64_t M, int64_t K,
                           void* stream) {
  if (!type_size(type)) return E_BAD_TYPE;
  if (!dtype_ok(dtype)) return E_BAD_DTYPE;
  if (M < 0 || K <= 0 || K % block_size(type) != 0) return E_BAD_SHAPE;
  if (M == 0) return E_OK;
  if (!X || !ws || !aligned16(ws) || !aligned16(X)) return E_BAD_POINTER;
  if (ws_bytes < q8_soa_bytes(M, K)) return E_WORKSPACE;
  return launch_quantize_q8_1(X, dtype, ws, M, K, Q8_MODE_SOA, gemv_sum_mode(type), 0, CORR_NONE, nullptr, 1, 0,
                              static_cast<cudaStream_t>(stream));
}

int gguf_b200_gemv_prepared(const void* W, const void* ws, void* Y, int type, int dtype, int64_t M, int64_t N,
                            int64_t K, void* stream) {
  int rc = check_common(W, ws, Y, type, dtype, M, N, K);
  if (rc || M == 0 || N == 0) return rc;
  int* st = status_ptr();
  if (!st) return E_CUDA;
  return launch_gemv(W, ws, Y, type, dtype, M, N, K, st, static_cast<cudaStream_t>(stream));
}

int gguf_b200_mul_mat_a8(const void* W, const void* X, void* Y, void* ws, int64_t ws_bytes, int type, int dtype,
                         int64_t M, int64_t N, int64_t K, void* stream) {
  int rc = check_common(W, X, Y, type, dtype, M, N, K);
  if (rc || M == 0 || N == 0) return rc;
  if (!is_mmq_type(type)) return E_BAD_TYPE;
  if (!ws || !aligned16(ws)) return E_BAD_POINTER;
  const int64_t ldb = mmq_ldb(type, K);
  if (ws_bytes < M * ldb * 2) return E_WORKSPACE;   // (always >= the GEMV scratch of the same M, K)
  int* st = status_ptr();
  if (!st) return E_CUDA;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (M <= mmq_gemv_max_tokens(type)) {
    // GEMV kernels with the tiled kernels' formulas: min / offset terms from the stored fp16 sum of the
    // inputs -- except Q5_0, whose tiled kernel folds the -16 into the codes (no sum term at all:
    // load_tiles_q5_0 + vec_dot_q8_0_q8_1_impl, vecdotq.cuh:676-749), i.e. 16 * d8 * sum(q8)
    rc = launch_quantize_q8_1(X, dtype, ws, M, K, Q8_MODE_SOA, type == T_Q5_0 ? 1 : 0, 0, CORR_NONE, nullptr, 1, 0, s);
    if (rc) return rc;
    return launch_gemv(W, ws, Y, type, dtype, M, N, K, st, s);
  }
  const int perm = mmq_perm(type, N, K, false, 0);
  rc = launch_quantize_q8_1(X, dtype, ws, M, K, Q8_MODE_F16, 0, ldb, mmq_corr_mode(type), nullptr, 1, 0, s, perm);
  if (rc) return rc;
  MmqArgs a{};
  a.perm = perm;
  a.w = W; a.b = ws; a.y = Y;
  a.type = type; a.out_dtype = dtype; a.b_dtype = DT_F16;
  a.M = M; a.N = N; a.K = K; a.ldb = ldb;
  a.corr_mode = mmq_corr_mode(type);
  a.rows_out = M;
  a.status = st;
  // whatever the caller gave beyond the activation matrix may hold split-K partial tiles
  const int64_t used = mmq_b_bytes(type, M, K);
  if (ws_bytes > used) {
    a.part = static_cast<uint8_t*>(ws) + used;
    a.part_bytes = ws_bytes - used;
  }
  return launch_mmq(a, s);
}

int gguf_b200_dequant_matmul(const void* W, const void* X, void* Y, void* ws, int64_t ws_bytes, int type, int dtype,
                             int64_t M, int64_t N, int64_t K, void* stream) {
  int rc = check_common(W, X, Y, type, dtype, M, N, K);
  if (rc || M == 0 || N == 0) return rc;
  if (type != T_IQ2_XXS && type != T_IQ4_XS && type != T_IQ4_NL) return E_BAD_TYPE;
  if (dtype != DT_F16 && dtype != DT_BF16) return E_BAD_DTYPE;
  if (K % 64 != 0) return E_BAD_SHAPE;
  int* st = status_ptr();
  if (!st) return E_CUDA;
  MmqArgs a{};
  a.w = W; a.b = X; a.y = Y;
  a.type = type; a.out_dtype = dtype; a.b_dtype = dtype;
  a.M = M; a.N = N; a.K = K; a.ldb = K;
  a.corr_mode = CORR_NONE;
  a.rows_out = M;
  a.status = st;
  if (ws && aligned16(ws) && ws_bytes > 0) {   // optional: room for split-K partial tiles
    a.part = ws;
    a.part_bytes = ws_bytes;
  }
  return launch_mmq(a, static_cast<cudaStream_t>(stream));
}

int gguf_b200_moe_a8(const void* X, const void* W, void* Y, void* ws, int64_t ws_bytes, const int32_t* sorted_token_ids,
                     const int32_t* expert_ids, const int32_t* num_tokens_post_padded, int64_t n_sorted,
                     int64_t expert_stride_bytes, int64_t n_experts, int type, int dtype, int64_t tokens, int64_t top_k,
                     int64_t N, int64_t K, void* stream) {
  int rc = check_common(W, X, Y, type, dtype, tokens, N, K);
  if (rc) return rc;
  if (!is_mmq_type(type)) return E_BAD_TYPE;
  if (top_k <= 0 || n_sorted < 0 || expert_stride_bytes % 16 != 0 || n_experts <= 0) return E_BAD_SHAPE;
  if (n_experts > 256) return E_TOO_LARGE;
  if (tokens == 0 || N == 0) return E_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t rows_out = tokens * top_k;
  const int64_t esz = dtype == DT_F32 ? 4 : 2;
  // rows that no routed token writes must read as zero (the reference allocates with new_zeros)
  if (cudaMemsetAsync(Y, 0, (size_t)(rows_out * N * esz), s) != cudaSuccess) return E_CUDA;
  if (n_sorted == 0) return E_OK;
  if (!sorted_token_ids || !expert_ids || !num_tokens_post_padded) return E_BAD_POINTER;
  if (!ws || !aligned16(ws)) return E_BAD_POINTER;
  const int64_t ldb = mmq_ldb(type, K);
  if (ws_bytes < n_sorted * ldb * 2) return E_WORKSPACE;
  int* st = status_ptr();
  if (!st) return E_CUDA;
  // quantize + gather: row p of the fp16 matrix = activations of token sorted_token_ids[p] / top_k
  const int perm = mmq_perm(type, N, K, true, expert_stride_bytes);
  rc = launch_quantize_q8_1(X, dtype, ws, n_sorted, K, Q8_MODE_F16, 0, ldb, mmq_corr_mode(type), sorted_token_ids, top_k,
                            rows_out, s, perm);
  if (rc) return rc;
  MmqArgs a{};
  a.perm = perm;
  a.w = W; a.b = ws; a.y = Y;
  a.type = type; a.out_dtype = dtype; a.b_dtype = DT_F16;
  a.M = n_sorted; a.N = N; a.K = K; a.ldb = ldb;
  a.corr_mode = mmq_corr_mode(type);
  a.sorted_ids = sorted_token_ids;
  a.expert_ids = expert_ids;
  a.n_post_pad = num_tokens_post_padded;
  a.n_sorted = n_sorted;
  a.expert_stride_bytes = expert_stride_bytes;
  a.top_k = top_k;
  a.rows_out = rows_out;
  a.n_experts = n_experts;
  a.moe_block = mmq_moe_block_size();
  a.status = st;
  return launch_mmq(a, s);
}

namespace {
struct FusedMoeLayout {
  int64_t n_sorted, o_counts, o_sorted, o_experts, o_npp, o_y1, o_y2, o_xb, total;
};
FusedMoeLayout fused_moe_layout(int type13, int type2, int dtype, int64_t tokens, int64_t top_k, int64_t E, int64_t H, int64_t I) {
  FusedMoeLayout L{};
  const int blk = mmq_moe_block_size();
  const int64_t slots = tokens * top_k, esz = dtype == DT_F32 ? 4 : 2;
  L.n_sorted = moe_align_sorted_len(slots, (int)E, blk);
  int64_t o = 0;
  auto take = [&](int64_t bytes) { const int64_t at = o; o += round_up(bytes, 256); return at; };
  L.o_counts = take(2 * E * 4);
  L.o_sorted = take(L.n_sorted * 4);
  L.o_experts = take(L.n_sorted / blk * 4);
  L.o_npp = take(4);
  L.o_y1 = take(slots * 2 * I * esz);
  L.o_y2 = take(slots * H * esz);
  const int64_t xb1 = L.n_sorted * mmq_ldb(type13, H) * 2, xb2 = L.n_sorted * mmq_ldb(type2, I) * 2;
  L.o_xb = take(xb1 > xb2 ? xb1 : xb2);
  L.total = o;
  return L;
}
}  // namespace

int64_t gguf_b200_fused_moe_workspace_bytes(int type13, int type2, int dtype, int64_t tokens, int64_t top_k, int64_t n_experts,
                                            int64_t H, int64_t I) {
  if (!is_mmq_type(type13) || !is_mmq_type(type2) || tokens < 0 || top_k <= 0 || n_experts <= 0 || n_experts > 256 || H <= 0 || I <= 0) return 0;
  return fused_moe_layout(type13, type2, dtype, tokens, top_k, n_experts, H, I).total;
}

int gguf_b200_fused_moe(const void* X, const void* W13, const void* W2, void* Y, const int32_t* topk_ids,
                        const float* topk_weights, void* ws, int64_t ws_bytes, int type13, int type2, int dtype, int act,
                        int64_t tokens, int64_t top_k, int64_t n_experts, int64_t H, int64_t I, void* stream) {
  int rc = check_common(W13, X, Y, type13, dtype, tokens, 2 * I, H);
  if (rc) return rc;
  rc = check_common(W2, X, Y, type2, dtype, tokens, H, I);
  if (rc) return rc;
  if (!is_mmq_type(type13) || !is_mmq_type(type2)) return E_BAD_TYPE;
  if (top_k <= 0 || n_experts <= 0 || (act != 1 && act != 2) || I % 8 != 0) return E_BAD_SHAPE;
  if (n_experts > 256) return E_TOO_LARGE;
  if (tokens == 0) return E_OK;
  if (!topk_ids || !topk_weights || !ws || !aligned16(ws)) return E_BAD_POINTER;
  const FusedMoeLayout L = fused_moe_layout(type13, type2, dtype, tokens, top_k, n_experts, H, I);
  if (ws_bytes < L.total) return E_WORKSPACE;
  int* st = status_ptr();
  if (!st) return E_CUDA;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint8_t* base = static_cast<uint8_t*>(ws);
  int32_t* sorted = reinterpret_cast<int32_t*>(base + L.o_sorted);
  int32_t* experts = reinterpret_cast<int32_t*>(base + L.o_experts);
  int32_t* npp = reinterpret_cast<int32_t*>(base + L.o_npp);
  void* y1 = base + L.o_y1;
  void* y2 = base + L.o_y2;
  void* xb = base + L.o_xb;
  const int64_t slots = tokens * top_k;
  const int blk = mmq_moe_block_size();
  // 1. expert-sorted, block-padded slot lists
  rc = launch_moe_align(topk_ids, slots, (int)n_experts, blk, reinterpret_cast<int32_t*>(base + L.o_counts), sorted, experts, npp, s);
  if (rc) return rc;
  // 2. gate/up projection of every routed slot.  Rows of y1 / y2 that belong to slots without a valid
  //    expert are never written and never read (the final sum skips them), so nothing is zero-filled.
  const int64_t rb13 = H / block_size(type13) * type_size(type13), rb2 = I / block_size(type2) * type_size(type2);
  auto gemm = [&](const void* x, int64_t x_rows_div, const void* w, int type, int64_t N, int64_t K, int64_t row_bytes, void* y,
                  const float* scale, int act_mode, int64_t x_ld) -> int {
    const int64_t ldb = mmq_ldb(type, K);
    const int64_t estride = N * row_bytes;
    const int perm = mmq_perm(type, N, K, true, estride);
    int r = launch_quantize_q8_1(x, dtype, xb, L.n_sorted, K, Q8_MODE_F16, 0, ldb, mmq_corr_mode(type), sorted, x_rows_div, slots, s,
                                 perm, nullptr, act_mode, x_ld);
    if (r) return r;
    MmqArgs a{};
    a.perm = perm;
    a.w = w; a.b = xb; a.y = y;
    a.type = type; a.out_dtype = dtype; a.b_dtype = DT_F16;
    a.M = L.n_sorted; a.N = N; a.K = K; a.ldb = ldb;
    a.corr_mode = mmq_corr_mode(type);
    a.sorted_ids = sorted;
    a.expert_ids = experts;
    a.n_post_pad = npp;
    a.n_sorted = L.n_sorted;
    a.expert_stride_bytes = estride;
    a.top_k = x_rows_div;
    a.rows_out = slots;
    a.n_experts = n_experts;
    a.moe_block = blk;
    a.row_scale = scale;
    a.status = st;
    return launch_mmq(a, s);
  };
  rc = gemm(X, top_k, W13, type13, 2 * I, H, rb13, y1, nullptr, 0, 0);
  if (rc) return rc;
  // 3. down projection: its activation quantizer applies act(gate) * up on the fly, its epilogue the routing weights
  rc = gemm(y1, 1, W2, type2, H, I, rb2, y2, topk_weights, act, 2 * I);
  if (rc) return rc;
  // 4. sum over the top_k slots of every token
  return launch_moe_sum(y2, Y, topk_ids, (int)n_experts, tokens, top_k, H, dtype, s);
}

int gguf_b200_moe_a8_vec(const void* X, const void* W, void* Y, void* ws, int64_t ws_bytes, const int32_t* topk_ids,
                         int64_t n_experts, int type, int dtype, int64_t tokens, int64_t top_k, int64_t N, int64_t K,
                         void* stream) {
  int rc = check_common(W, X, Y, type, dtype, tokens, N, K);
  if (rc || tokens == 0 || N == 0) return rc;
  if (top_k <= 0 || n_experts <= 0) return E_BAD_SHAPE;
  if (!topk_ids || !ws || !aligned16(ws)) return E_BAD_POINTER;
  if (ws_bytes < q8_soa_bytes(tokens, K)) return E_WORKSPACE;
  int* st = status_ptr();
  if (!st) return E_CUDA;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  rc = launch_quantize_q8_1(X, dtype, ws, tokens, K, Q8_MODE_SOA, gemv_sum_mode(type), 0, CORR_NONE, nullptr, 1, 0, s);
  if (rc) return rc;
  return launch_moe_gemv(W, ws, Y, topk_ids, type, dtype, tokens, top_k, N, K, n_experts, st, s);
}

}  // extern "C"
