// Decode GEMV for callers that cannot give the library a workspace.
//
// Every other matmul entry point takes its scratch memory from the caller.  Some hosts cannot
// provide one: a plain-C / FFI integration (cgo, ctypes, a C++ engine plug-in) that is handed
// only the W, X and Y pointers, inside an inference engine that has claimed the whole device
// for weights and KV cache at start-up.  Such a caller has no pool to carve a workspace from,
// and a cudaMalloc at that point may fail or fragment what the engine reserved -- so it must
// not allocate at all.  This file gives those callers one GEMV entry point whose scratch (the
// q8_1-quantized activations) lives in a fixed array inside the library image.
//
// The array is `static __device__`: every GPU that loads the library holds its
// GGUF_B200_NOALLOC_SCRATCH_BYTES (320 KiB) until the process exits.  In host code the array's
// name is only a handle, not a device address; the address is looked up once per device with
// cudaGetSymbolAddress while that device is current, and that pointer is what the kernels get.
#include "../../include/gguf_b200.h"

#include "common.cuh"
#include "kernels.h"

using namespace gguf_b200;

namespace {

// room for 8 vectors of K = 32768: 8 * (32768 int8 codes + 1024 * 8 bytes of {d, sum})
constexpr int64_t kScratchBytes = 8 * (32768 + 32768 / 4);
constexpr int64_t kMaxVectors = 8;
constexpr int64_t kMaxK = 32768;

static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

struct DevicePtrs {
  void* scratch = nullptr;
  int* status = nullptr;
};

// Set-up, once per device, with that device current: resolve the device address of the
// file-scope scratch array, and take the library's one status word (the word that
// gguf_b200_last_status reads), so that a bounded wait that expires in these kernels is reported
// exactly as for every other entry point.  Returns false if the runtime refuses.
bool device_ptrs(DevicePtrs& out) {
  static DevicePtrs cache[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
  DevicePtrs& c = cache[dev];
  if (!c.scratch) {
    void* s = nullptr;
    if (cudaGetSymbolAddress(&s, g_noalloc_scratch) != cudaSuccess || !s) return false;
    int* st = status_word_ptr();
    if (!st) return false;
    c.status = st;
    c.scratch = s;
  }
  out = c;
  return true;
}

}  // namespace

extern "C" {

int64_t gguf_b200_noalloc_scratch_bytes(void) { return kScratchBytes; }

int gguf_b200_mul_mat_vec_a8_noalloc(const void* W, const void* X, void* Y, int type, int dtype, int64_t M, int64_t N,
                                     int64_t K, void* stream) {
  if (!type_size(type)) return E_BAD_TYPE;
  if (dtype != DT_F32 && dtype != DT_F16 && dtype != DT_BF16) return E_BAD_DTYPE;
  if (M < 0 || N < 0 || K <= 0 || K % block_size(type) != 0) return E_BAD_SHAPE;
  if (M > kMaxVectors || K > kMaxK || q8_soa_bytes(M, K) > kScratchBytes) return E_TOO_LARGE;
  if (M == 0 || N == 0) return E_OK;
  auto a16 = [](const void* p) { return p && (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (!a16(W) || !a16(X) || !a16(Y)) return E_BAD_POINTER;
  DevicePtrs dp;
  if (!device_ptrs(dp)) return E_CUDA;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // The quantizer rewrites every byte of the scratch that the GEMV will read (codes up to the
  // padded K and one {d, sum} pair per 32), so nothing has to be cleared between calls.
  int rc = launch_quantize_q8_1(X, dtype, dp.scratch, M, K, Q8_MODE_SOA, gemv_sum_mode(type), 0, CORR_NONE, nullptr, 1, 0, s);
  if (rc) return rc;
  return launch_gemv(W, dp.scratch, Y, type, dtype, M, N, K, dp.status, s);
}

}  // extern "C"
