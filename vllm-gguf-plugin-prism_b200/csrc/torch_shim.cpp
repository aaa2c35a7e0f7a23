// Torch library `_C_gguf` over the C-ABI of libgguf_b200: the six operator schemas of the
// reference's binding file (vllm_gguf_plugin/csrc/torch_bindings.cpp:22-53), registered the
// same way (stable ABI, five ops on the CUDA key, ggml_moe_get_block_size as
// CompositeExplicitAutograd), so `vllm_gguf_plugin.ops` finds `torch.ops._C_gguf.*` unchanged.
// This file only validates tensors, allocates the output and the scratch tensor from torch's
// caching allocator (so CUDA-graph capture works as in the reference), resolves the current
// stream and turns error codes into exceptions.  All arithmetic lives behind gguf_b200.h.
// One more op, dequant_matmul, exposes the fused route for the IQ types.
#include <optional>
#include <string>

#include <Python.h>
#include <torch/csrc/inductor/aoti_torch/c/shim.h>
#include <torch/csrc/stable/accelerator.h>
#include <torch/csrc/stable/library.h>
#include <torch/csrc/stable/ops.h>
#include <torch/csrc/stable/tensor.h>
#include <torch/headeronly/core/ScalarType.h>

#include "../../include/gguf_b200.h"

using torch::headeronly::ScalarType;
using torch::stable::Tensor;
using torch::stable::accelerator::DeviceGuard;

namespace {

void* current_stream(int32_t device_index) {
  void* raw = nullptr;
  TORCH_ERROR_CODE_CHECK(aoti_torch_get_current_cuda_stream(device_index, &raw));
  return raw;
}

int dtype_code(ScalarType t, const char* what) {
  switch (t) {
    case ScalarType::Float: return GGUF_B200_F32;
    case ScalarType::Half: return GGUF_B200_F16;
    case ScalarType::BFloat16: return GGUF_B200_BF16;
    default: break;
  }
  STD_TORCH_CHECK(false, what, ": expected a float32, float16 or bfloat16 tensor");
  return -1;
}

void check_rc(int rc, const char* op) {
  STD_TORCH_CHECK(rc == GGUF_B200_OK, op, " failed: ", gguf_b200_error_string(rc));
}

// Weights are raw GGUF bytes: uint8, contiguous, last dim a whole number of blocks.
int64_t check_weight(const Tensor& W, int64_t type, const char* op) {
  const int ts = gguf_b200_type_size((int)type);
  STD_TORCH_CHECK(ts > 0, op, ": unsupported GGML quantization type ", std::to_string(type));
  STD_TORCH_CHECK(W.scalar_type() == ScalarType::Byte, op, ": W must be a uint8 tensor of raw GGUF blocks");
  STD_TORCH_CHECK(W.is_contiguous(), op, ": W must be contiguous");
  STD_TORCH_CHECK(W.dim() >= 1 && W.size(W.dim() - 1) % ts == 0, op, ": last dim of W is not a whole number of blocks");
  return W.size(W.dim() - 1) / ts * gguf_b200_block_size((int)type);  // K
}

Tensor scratch(const Tensor& like, int64_t bytes) {
  return torch::stable::new_empty(like, {bytes > 0 ? bytes : 1}, ScalarType::Byte);
}

}  // namespace

Tensor ggml_dequantize(Tensor W, int64_t type, int64_t m, int64_t n, std::optional<ScalarType> dtype) {
  const int32_t dev = W.get_device_index();
  const DeviceGuard guard(dev);
  check_weight(W, type, "ggml_dequantize");
  const ScalarType dt = dtype.value_or(ScalarType::Half);
  const int code = dtype_code(dt, "ggml_dequantize");
  const int ts = gguf_b200_type_size((int)type), bs = gguf_b200_block_size((int)type);
  STD_TORCH_CHECK(m >= 0 && n >= 0 && (m * n) % bs == 0, "ggml_dequantize: m*n must be a multiple of the block size");
  STD_TORCH_CHECK(W.numel() >= m * n / bs * ts, "ggml_dequantize: W holds fewer than m*n values");
  Tensor out = torch::stable::new_empty(W, {m, n}, dt);  // every element is written by the kernel
  check_rc(gguf_b200_dequantize(W.data_ptr(), (int)type, out.data_ptr(), code, m * n, current_stream(dev)), "ggml_dequantize");
  return out;
}

// Embedding look-up: rows `ids` of the packed weight, dequantized (replaces index_select +
// ggml_dequantize of the reference's embedding caller, quantization/vocal_embeds.py:88-96).
Tensor dequantize_rows(Tensor W, Tensor ids, int64_t type, std::optional<ScalarType> dtype) {
  const int32_t dev = W.get_device_index();
  const DeviceGuard guard(dev);
  const int64_t K = check_weight(W, type, "dequantize_rows");
  STD_TORCH_CHECK(W.dim() == 2, "dequantize_rows: W must be [rows, bytes]");
  STD_TORCH_CHECK(ids.scalar_type() == ScalarType::Long && ids.is_contiguous() && ids.dim() == 1,
                  "dequantize_rows: ids must be a contiguous 1-D int64 tensor");
  STD_TORCH_CHECK(K % 256 == 0, "dequantize_rows: the row length must be a multiple of 256");
  const ScalarType dt = dtype.value_or(ScalarType::Half);
  const int code = dtype_code(dt, "dequantize_rows");
  Tensor out = torch::stable::new_empty(W, {ids.size(0), K}, dt);
  check_rc(gguf_b200_dequantize_rows(W.data_ptr(), (int)type, static_cast<const int64_t*>(ids.data_ptr()), ids.size(0), K,
                                     W.size(0), out.data_ptr(), code, current_stream(dev)),
           "dequantize_rows");
  return out;
}

static Tensor matmul_common(const Tensor& W, const Tensor& X, int64_t type, int64_t row, int op, const char* name) {
  const int32_t dev = X.get_device_index();
  const DeviceGuard guard(dev);
  const int64_t K = check_weight(W, type, name);
  STD_TORCH_CHECK(X.dim() == 2 && X.is_contiguous(), name, ": X must be a contiguous [tokens, K] tensor");
  STD_TORCH_CHECK(X.size(1) == K, name, ": X.shape[1] does not match the K implied by W");
  STD_TORCH_CHECK(row >= 0 && W.numel() / W.size(W.dim() - 1) >= row, name, ": W has fewer than `row` rows");
  const int code = dtype_code(X.scalar_type(), name);
  const int64_t M = X.size(0);
  Tensor Y = torch::stable::new_empty(W, {M, row}, X.scalar_type());
  if (M == 0 || row == 0) return Y;
  const int64_t ws_bytes = gguf_b200_workspace_bytes(op, (int)type, M, row, K);
  Tensor ws = scratch(W, ws_bytes);
  void* s = current_stream(dev);
  int rc;
  if (op == GGUF_B200_OP_GEMV)
    rc = gguf_b200_mul_mat_vec_a8(W.data_ptr(), X.data_ptr(), Y.data_ptr(), ws.data_ptr(), ws_bytes, (int)type, code, M, row, K, s);
  else if (op == GGUF_B200_OP_MMQ)
    rc = gguf_b200_mul_mat_a8(W.data_ptr(), X.data_ptr(), Y.data_ptr(), ws.data_ptr(), ws_bytes, (int)type, code, M, row, K, s);
  else
    rc = gguf_b200_dequant_matmul(W.data_ptr(), X.data_ptr(), Y.data_ptr(), ws.data_ptr(), ws_bytes, (int)type, code, M, row, K, s);
  check_rc(rc, name);
  return Y;
}

Tensor ggml_mul_mat_vec_a8(Tensor W, Tensor X, int64_t type, int64_t row) {
  return matmul_common(W, X, type, row, GGUF_B200_OP_GEMV, "ggml_mul_mat_vec_a8");
}
Tensor ggml_mul_mat_a8(Tensor W, Tensor X, int64_t type, int64_t row) {
  return matmul_common(W, X, type, row, GGUF_B200_OP_MMQ, "ggml_mul_mat_a8");
}
Tensor dequant_matmul(Tensor W, Tensor X, int64_t type, int64_t row) {
  return matmul_common(W, X, type, row, GGUF_B200_OP_DEQUANT_MATMUL, "dequant_matmul");
}

Tensor ggml_moe_a8(Tensor X, Tensor W, Tensor sorted_token_ids, Tensor expert_ids, Tensor num_tokens_post_padded,
                   int64_t type, int64_t row, int64_t top_k, int64_t tokens) {
  const int32_t dev = X.get_device_index();
  const DeviceGuard guard(dev);
  const int64_t K = check_weight(W, type, "ggml_moe_a8");
  STD_TORCH_CHECK(W.dim() == 3, "ggml_moe_a8: W must be [experts, rows, bytes]");
  STD_TORCH_CHECK(X.dim() == 2 && X.is_contiguous() && X.size(1) == K, "ggml_moe_a8: X must be contiguous [tokens, K]");
  STD_TORCH_CHECK(X.size(0) == tokens, "ggml_moe_a8: X.shape[0] != tokens");
  STD_TORCH_CHECK(row == W.size(1), "ggml_moe_a8: row != W.shape[1]");
  STD_TORCH_CHECK(sorted_token_ids.scalar_type() == ScalarType::Int && expert_ids.scalar_type() == ScalarType::Int &&
                      num_tokens_post_padded.scalar_type() == ScalarType::Int,
                  "ggml_moe_a8: routing tensors must be int32");
  STD_TORCH_CHECK(sorted_token_ids.is_contiguous() && expert_ids.is_contiguous(), "ggml_moe_a8: routing tensors must be contiguous");
  const int blk = gguf_b200_moe_block_size((int)type);
  STD_TORCH_CHECK(blk > 0, "ggml_moe_a8: type has no tensor-core MoE kernel");
  const int64_t n_sorted = sorted_token_ids.numel();
  // vLLM sizes sorted_token_ids as numel + E*(block-1) (not rounded) and expert_ids as its ceil-div by block
  STD_TORCH_CHECK(expert_ids.numel() * blk >= n_sorted,
                  "ggml_moe_a8: sorted_token_ids/expert_ids were not built with block size ggml_moe_get_block_size(type)");
  const int code = dtype_code(X.scalar_type(), "ggml_moe_a8");
  Tensor Y = torch::stable::new_empty(W, {tokens * top_k, row}, X.scalar_type());  // zeroed by the C-ABI call
  const int64_t ws_bytes = gguf_b200_workspace_bytes(GGUF_B200_OP_MOE, (int)type, n_sorted, row, K);
  Tensor ws = scratch(W, ws_bytes);
  check_rc(gguf_b200_moe_a8(X.data_ptr(), W.data_ptr(), Y.data_ptr(), ws.data_ptr(), ws_bytes,
                            static_cast<const int32_t*>(sorted_token_ids.data_ptr()),
                            static_cast<const int32_t*>(expert_ids.data_ptr()),
                            static_cast<const int32_t*>(num_tokens_post_padded.data_ptr()), n_sorted, W.stride(0),
                            W.size(0) < 256 ? W.size(0) : 256,   // ids beyond 255 are skipped, as in the reference (moe.cuh:33)
                            (int)type, code, tokens, top_k, row, K, current_stream(dev)),
           "ggml_moe_a8");
  return Y;
}

Tensor ggml_moe_a8_vec(Tensor X, Tensor W, Tensor topk_ids, int64_t top_k, int64_t type, int64_t row, int64_t tokens) {
  const int32_t dev = X.get_device_index();
  const DeviceGuard guard(dev);
  const int64_t K = check_weight(W, type, "ggml_moe_a8_vec");
  STD_TORCH_CHECK(W.dim() == 3 && row == W.size(1), "ggml_moe_a8_vec: W must be [experts, row, bytes]");
  STD_TORCH_CHECK(X.dim() == 2 && X.is_contiguous() && X.size(1) == K && X.size(0) == tokens,
                  "ggml_moe_a8_vec: X must be contiguous [tokens, K]");
  STD_TORCH_CHECK(topk_ids.scalar_type() == ScalarType::Int && topk_ids.is_contiguous() && topk_ids.numel() == tokens * top_k,
                  "ggml_moe_a8_vec: topk_ids must be contiguous int32 [tokens, top_k]");
  const int code = dtype_code(X.scalar_type(), "ggml_moe_a8_vec");
  Tensor Y = torch::stable::new_empty(W, {tokens * top_k, row}, X.scalar_type());
  if (tokens == 0 || row == 0) return Y;
  const int64_t ws_bytes = gguf_b200_workspace_bytes(GGUF_B200_OP_MOE_VEC, (int)type, tokens, row, K);
  Tensor ws = scratch(W, ws_bytes);
  check_rc(gguf_b200_moe_a8_vec(X.data_ptr(), W.data_ptr(), Y.data_ptr(), ws.data_ptr(), ws_bytes,
                                static_cast<const int32_t*>(topk_ids.data_ptr()), W.size(0), (int)type, code, tokens,
                                top_k, row, K, current_stream(dev)),
           "ggml_moe_a8_vec");
  return Y;
}

// The tiled MoE step in one call (see gguf_b200_fused_moe).  act: 1 silu, 2 gelu.
Tensor fused_moe(Tensor X, Tensor W13, Tensor W2, Tensor topk_weights, Tensor topk_ids, int64_t type13, int64_t type2, int64_t act) {
  const int32_t dev = X.get_device_index();
  const DeviceGuard guard(dev);
  const int64_t H = check_weight(W13, type13, "fused_moe");
  const int64_t I = check_weight(W2, type2, "fused_moe");
  STD_TORCH_CHECK(W13.dim() == 3 && W2.dim() == 3 && W13.size(0) == W2.size(0), "fused_moe: W13 / W2 must be [experts, rows, bytes]");
  STD_TORCH_CHECK(W13.size(1) == 2 * I && W2.size(1) == H, "fused_moe: W13 must be [E, 2I, .] and W2 [E, H, .]");
  STD_TORCH_CHECK(X.dim() == 2 && X.is_contiguous() && X.size(1) == H, "fused_moe: X must be contiguous [tokens, H]");
  STD_TORCH_CHECK(topk_ids.scalar_type() == ScalarType::Int && topk_ids.is_contiguous() && topk_ids.dim() == 2 && topk_ids.size(0) == X.size(0),
                  "fused_moe: topk_ids must be contiguous int32 [tokens, top_k]");
  STD_TORCH_CHECK(topk_weights.scalar_type() == ScalarType::Float && topk_weights.is_contiguous() && topk_weights.numel() == topk_ids.numel(),
                  "fused_moe: topk_weights must be contiguous float32 [tokens, top_k]");
  const int code = dtype_code(X.scalar_type(), "fused_moe");
  const int64_t tokens = X.size(0), top_k = topk_ids.size(1), E = W13.size(0);
  Tensor Y = torch::stable::new_empty(X, {tokens, H}, X.scalar_type());
  const int64_t ws_bytes = gguf_b200_fused_moe_workspace_bytes((int)type13, (int)type2, code, tokens, top_k, E, H, I);
  STD_TORCH_CHECK(ws_bytes > 0 || tokens == 0, "fused_moe: unsupported types or sizes");
  Tensor ws = scratch(X, ws_bytes);
  check_rc(gguf_b200_fused_moe(X.data_ptr(), W13.data_ptr(), W2.data_ptr(), Y.data_ptr(), static_cast<const int32_t*>(topk_ids.data_ptr()),
                               static_cast<const float*>(topk_weights.data_ptr()), ws.data_ptr(), ws_bytes, (int)type13, (int)type2, code,
                               (int)act, tokens, top_k, E, H, I, current_stream(dev)),
           "fused_moe");
  return Y;
}

int64_t ggml_moe_get_block_size(int64_t type) { return gguf_b200_moe_block_size((int)type); }

STABLE_TORCH_LIBRARY(_C_gguf, ops) {
  ops.def("ggml_dequantize(Tensor W, int type, SymInt m, SymInt n, ScalarType? dtype) -> Tensor");
  ops.def("ggml_mul_mat_vec_a8(Tensor W, Tensor X, int type, SymInt row) -> Tensor");
  ops.def("ggml_mul_mat_a8(Tensor W, Tensor X, int type, SymInt row) -> Tensor");
  ops.def(
      "ggml_moe_a8(Tensor X, Tensor W, Tensor sorted_token_ids, Tensor expert_ids, Tensor num_tokens_post_padded, "
      "int type, SymInt row, SymInt top_k, SymInt tokens) -> Tensor");
  ops.def("ggml_moe_a8_vec(Tensor X, Tensor W, Tensor topk_ids, int top_k, int type, SymInt row, SymInt tokens) -> Tensor");
  ops.def("ggml_moe_get_block_size(int type) -> int");
  ops.def("dequant_matmul(Tensor W, Tensor X, int type, SymInt row) -> Tensor");
  ops.def("dequantize_rows(Tensor W, Tensor ids, int type, ScalarType? dtype) -> Tensor");
  ops.def("fused_moe(Tensor X, Tensor W13, Tensor W2, Tensor topk_weights, Tensor topk_ids, int type13, int type2, int act) -> Tensor");
}

STABLE_TORCH_LIBRARY_IMPL(_C_gguf, CUDA, ops) {
  ops.impl("ggml_dequantize", TORCH_BOX(&ggml_dequantize));
  ops.impl("ggml_mul_mat_vec_a8", TORCH_BOX(&ggml_mul_mat_vec_a8));
  ops.impl("ggml_mul_mat_a8", TORCH_BOX(&ggml_mul_mat_a8));
  ops.impl("ggml_moe_a8", TORCH_BOX(&ggml_moe_a8));
  ops.impl("ggml_moe_a8_vec", TORCH_BOX(&ggml_moe_a8_vec));
  ops.impl("dequant_matmul", TORCH_BOX(&dequant_matmul));
  ops.impl("dequantize_rows", TORCH_BOX(&dequantize_rows));
  ops.impl("fused_moe", TORCH_BOX(&fused_moe));
}

STABLE_TORCH_LIBRARY_IMPL(_C_gguf, CompositeExplicitAutograd, ops) {
  ops.impl("ggml_moe_get_block_size", TORCH_BOX(&ggml_moe_get_block_size));
}

static struct PyModuleDef gguf_module_def = {PyModuleDef_HEAD_INIT, "_C_gguf", nullptr, -1, nullptr};

extern "C" PyObject* PyInit__C_gguf(void) { return PyModule_Create(&gguf_module_def); }
