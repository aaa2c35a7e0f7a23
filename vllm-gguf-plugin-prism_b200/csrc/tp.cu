// Consumer side of the tensor-parallel entry points: the kernels that wait for what the other
// ranks' GPUs write into this rank's memory.
//
//  * Decode (one vector, gguf_b200_mul_mat_vec_a8_tp): the GEMV kernels of all ranks send every
//    output element as a tagged packet (common.cuh, packet_read).  tp_unpack_kernel turns the
//    packets of one or several gathered vectors into plain vectors, polling each packet until
//    its tag is the expected launch number.  (The next decode GEMV can also read the packets
//    itself, in its activation quantizer: quantize_q8_1.cu.)
//  * Prefill (gguf_b200_matmul_tp): the GEMM kernels store their tiles into every rank's output
//    matrix and the last CTA of each rank raises a per-call flag on every rank (mmq.cu,
//    tp_finish).  tp_wait_kernel is the one-thread kernel that waits for `world` raises.
//
// Both waits are bounded by a caller-settable number of SM clock cycles
// (gguf_b200_set_wait_limit_cycles); when it runs out the kernel records E_TIMEOUT in the status
// word and returns -- the context stays usable, nothing hangs.
#include "common.cuh"
#include "kernels.h"

namespace gguf_b200 {

__global__ void tp_wait_kernel(const unsigned* flag, const unsigned* epoch, int slot, int world, long long limit_cycles, int* status) {
  pdl_trigger();   // whatever follows may be scheduled; it waits for this grid before it reads
  pdl_wait();      // this rank's own kernels before this one have finished
  const unsigned want = epoch[slot] * (unsigned)world;
  const long long t0 = clock64();
  for (;;) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag + slot) : "memory");
    if ((int)(v - want) >= 0) return;
    if (clock64() - t0 > limit_cycles) {   // a rank is missing
      atomicExch(status, E_TIMEOUT);
      return;
    }
  }
}

int launch_tp_wait(const unsigned* flag, const unsigned* epoch, int slot, int world, long long limit_cycles, int* status,
                   cudaStream_t stream) {
  return launch_pdl(tp_wait_kernel, dim3(1), dim3(1), 0, stream, flag, epoch, slot, world, limit_cycles, status) == cudaSuccess ? E_OK : E_CUDA;
}

template <typename T>
__global__ void __launch_bounds__(256) tp_unpack_kernel(const void* packets, const unsigned* epoch, int slot0, int64_t slot_packets,
                                                        int64_t n, T* out, int64_t out_stride, long long limit_cycles, int* status) {
  pdl_trigger();
  pdl_wait();
  const int s = blockIdx.y;
  const unsigned want = epoch[slot0 + s];
  const char* base = static_cast<const char*>(packets) + (int64_t)(slot0 + s) * slot_packets * (sizeof(T) == 2 ? 4 : 8);
  bool ok = true;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    float v;
    if (ok) {
      ok = packet_read<T>(base, i, want, limit_cycles, v);
    } else {   // this thread already gave up once: do not spend the limit again on every element
      packet_read<T>(base, i, want, 0, v);
    }
    out[(int64_t)s * out_stride + i] = from_float<T>(v);   // exact: the packet carries the T value
  }
  if (!ok) atomicExch(status, E_TIMEOUT);
}

// All-reduce side of a row-parallel call: the slot holds `parts` fp32 partial vectors (one per rank,
// n packets apart); out[i] = their sum in rank order -- the same order on every rank, so all ranks
// hold identical bits -- rounded once to T.
template <typename T>
__global__ void __launch_bounds__(256) tp_unpack_sum_kernel(const void* packets, const unsigned* epoch, int slot, int64_t slot_bytes,
                                                            int64_t n, int parts, T* out, long long limit_cycles, int* status) {
  pdl_trigger();
  pdl_wait();
  const unsigned want = epoch[slot];
  const char* base = static_cast<const char*>(packets) + (int64_t)slot * slot_bytes;
  bool ok = true;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    float s = 0.f;
    for (int r = 0; r < parts; ++r) {
      float v;
      ok = packet_read<float>(base, (int64_t)r * n + i, want, ok ? limit_cycles : 0, v) && ok;
      s += v;
    }
    out[i] = from_float<T>(s);
  }
  if (!ok) atomicExch(status, E_TIMEOUT);
}

int launch_tp_unpack_sum(const void* packets, const unsigned* epoch, int slot, int64_t slot_bytes, int64_t n, int parts, void* out,
                         int dtype, long long limit_cycles, int* status, cudaStream_t stream) {
  if (n <= 0) return E_OK;
  const int64_t want = (n + 255) / 256;
  const dim3 grid((unsigned)(want > 148 ? 148 : want));
  cudaError_t e;
  switch (dtype) {
    case DT_F32:
      e = launch_pdl(tp_unpack_sum_kernel<float>, grid, dim3(256), 0, stream, packets, epoch, slot, slot_bytes, n, parts, static_cast<float*>(out), limit_cycles, status);
      break;
    case DT_F16:
      e = launch_pdl(tp_unpack_sum_kernel<__half>, grid, dim3(256), 0, stream, packets, epoch, slot, slot_bytes, n, parts, static_cast<__half*>(out), limit_cycles, status);
      break;
    case DT_BF16:
      e = launch_pdl(tp_unpack_sum_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, packets, epoch, slot, slot_bytes, n, parts, static_cast<__nv_bfloat16*>(out), limit_cycles, status);
      break;
    default:
      return E_BAD_DTYPE;
  }
  return e == cudaSuccess ? E_OK : E_CUDA;
}

int launch_tp_unpack(const void* packets, const unsigned* epoch, int slot0, int nslots, int64_t slot_packets, int64_t n,
                     void* out, int64_t out_stride, int dtype, long long limit_cycles, int* status, cudaStream_t stream) {
  if (nslots <= 0 || n <= 0) return E_OK;
  if (nslots > 65535) return E_TOO_LARGE;
  const int64_t want = (n + 255) / 256;
  const dim3 grid((unsigned)(want > 148 ? 148 : want), (unsigned)nslots);
  cudaError_t e;
  switch (dtype) {
    case DT_F32:
      e = launch_pdl(tp_unpack_kernel<float>, grid, dim3(256), 0, stream, packets, epoch, slot0, slot_packets, n, static_cast<float*>(out), out_stride, limit_cycles, status);
      break;
    case DT_F16:
      e = launch_pdl(tp_unpack_kernel<__half>, grid, dim3(256), 0, stream, packets, epoch, slot0, slot_packets, n, static_cast<__half*>(out), out_stride, limit_cycles, status);
      break;
    case DT_BF16:
      e = launch_pdl(tp_unpack_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, packets, epoch, slot0, slot_packets, n, static_cast<__nv_bfloat16*>(out), out_stride, limit_cycles, status);
      break;
    default:
      return E_BAD_DTYPE;
  }
  return e == cudaSuccess ? E_OK : E_CUDA;
}

}  // namespace gguf_b200
