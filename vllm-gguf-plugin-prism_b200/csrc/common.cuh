// Shared device helpers of the B200 GGUF kernels: block geometry of the six supported
// formats, typed stores, bounded mbarrier waits and the 1-D bulk (TMA) copy used to
// stream packed weight bytes into shared memory.
//
// Block layouts (bytes), as defined by the GGUF format and used by the reference at
// vllm_gguf_plugin/csrc/gguf/ggml-common.h:17-23 (Q4_0), :51-57 (Q8_0), :84-90 (Q4_K),
// :101-108 (Q6_K), :110-115 (IQ2_XXS), :184-191 (IQ4_XS), :59-65 (q8_1 activations):
//   Q4_0    18 : half d | u8 qs[16]            value j = qs[j]&15, value j+16 = qs[j]>>4, minus 8
//   Q8_0    34 : half d | i8 qs[32]
//   Q4_K   144 : half d | half dmin | u8 scales[12] | u8 qs[128]
//   Q6_K   210 : u8 ql[128] | u8 qh[64] | i8 scales[16] | half d
//   IQ2_XXS 66 : half d | u16 qs[32]           per 32 values: 4 grid indices + 28 sign bits + 4-bit scale
//   IQ4_XS 136 : half d | u16 scales_h | u8 scales_l[4] | u8 qs[128]
//   q8_1    36 : half d | half sum | i8 qs[32]
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

namespace gguf_b200 {

enum : int { T_Q4_0 = 2, T_Q8_0 = 8, T_Q4_K = 12, T_Q6_K = 14, T_IQ2_XXS = 16, T_IQ4_XS = 23 };
// further block types (Q2_K, Q3_K: dequantize and GEMV):
//   Q4_1    20 : half d | half m | u8 qs[16]                      value = q*d + m
//   Q5_0    22 : half d | u8 qh[4] | u8 qs[16]                    5th bit of value j in bit j (j+16: bit j+16... see dequantize.cu)
//   Q5_1    24 : half d | half m | u8 qh[4] | u8 qs[16]
//   Q2_K    84 : u8 scales[16] | u8 qs[64] | half d | half dmin
//   Q3_K   110 : u8 hmask[32] | u8 qs[64] | u8 scales[12] | half d
//   Q5_K   176 : half d | half dmin | u8 scales[12] | u8 qh[32] | u8 qs[128]
//   IQ4_NL  18 : half d | u8 qs[16]                               4-bit indices into the IQ4 level table
enum : int { T_Q4_1 = 3, T_Q5_0 = 6, T_Q5_1 = 7, T_Q2_K = 10, T_Q3_K = 11, T_Q5_K = 13, T_IQ4_NL = 20 };
// code-book types served by the dequantizer and the decode GEMV (256 values per block; for more
// tokens the callers dequantize and then multiply, as the reference does above its GEMV threshold):
//   IQ2_XS   74 : half d | u16 qs[32] | u8 scales[8]
//   IQ2_S    82 : half d | u8 qs[32] | u8 signs[32] | u8 qh[8] | u8 scales[8]
//   IQ3_XXS  98 : half d | u8 qs[64] | u32 scales_and_signs[8]
//   IQ3_S   110 : half d | u8 qs[64] | u8 qh[8] | u8 signs[32] | u8 scales[4]
//   IQ1_S    50 : half d | u8 qs[32] | u16 qh[8]
//   IQ1_M    56 : u8 qs[32] | u8 qh[16] | u8 scales[8]   (the fp16 scale is spread over the top nibbles of scales)
enum : int { T_IQ2_XS = 17, T_IQ3_XXS = 18, T_IQ1_S = 19, T_IQ3_S = 21, T_IQ2_S = 22, T_IQ1_M = 29 };
enum : int { DT_F32 = 0, DT_F16 = 1, DT_BF16 = 2 };

// error codes returned through the C-ABI (0 = success)
enum : int {
  E_OK = 0,
  E_BAD_TYPE = -1,      // block type not one of the six supported
  E_BAD_DTYPE = -2,     // activation/output dtype not f32/f16/bf16
  E_BAD_SHAPE = -3,     // K not a multiple of the block size, negative sizes, ...
  E_BAD_POINTER = -4,   // null or insufficiently aligned pointer
  E_WORKSPACE = -5,     // scratch buffer smaller than gguf_b200_workspace_bytes()
  E_CUDA = -6,          // a CUDA runtime call failed (see cudaGetLastError)
  E_TOO_LARGE = -7,     // size beyond what the entry point supports
  E_TIMEOUT = -8,       // a bounded device-side wait ran out (status word set by the kernel)
};

template <int TYPE> struct BlockTraits;
template <> struct BlockTraits<T_Q4_0>    { static constexpr int QK = 32,  TS = 18;  };
template <> struct BlockTraits<T_Q8_0>    { static constexpr int QK = 32,  TS = 34;  };
template <> struct BlockTraits<T_Q4_K>    { static constexpr int QK = 256, TS = 144; };
template <> struct BlockTraits<T_Q6_K>    { static constexpr int QK = 256, TS = 210; };
template <> struct BlockTraits<T_IQ2_XXS> { static constexpr int QK = 256, TS = 66;  };
template <> struct BlockTraits<T_IQ4_XS>  { static constexpr int QK = 256, TS = 136; };
template <> struct BlockTraits<T_Q4_1>    { static constexpr int QK = 32,  TS = 20;  };
template <> struct BlockTraits<T_Q5_0>    { static constexpr int QK = 32,  TS = 22;  };
template <> struct BlockTraits<T_Q5_1>    { static constexpr int QK = 32,  TS = 24;  };
template <> struct BlockTraits<T_Q2_K>    { static constexpr int QK = 256, TS = 84;  };
template <> struct BlockTraits<T_Q3_K>    { static constexpr int QK = 256, TS = 110; };
template <> struct BlockTraits<T_Q5_K>    { static constexpr int QK = 256, TS = 176; };
template <> struct BlockTraits<T_IQ4_NL>  { static constexpr int QK = 32,  TS = 18;  };
template <> struct BlockTraits<T_IQ2_XS>  { static constexpr int QK = 256, TS = 74;  };
template <> struct BlockTraits<T_IQ2_S>   { static constexpr int QK = 256, TS = 82;  };
template <> struct BlockTraits<T_IQ3_XXS> { static constexpr int QK = 256, TS = 98;  };
template <> struct BlockTraits<T_IQ3_S>   { static constexpr int QK = 256, TS = 110; };
template <> struct BlockTraits<T_IQ1_S>   { static constexpr int QK = 256, TS = 50;  };
template <> struct BlockTraits<T_IQ1_M>   { static constexpr int QK = 256, TS = 56;  };

// block geometry of the types the matmul entry points take
__host__ __device__ inline int type_size(int t) {
  switch (t) {
    case T_Q4_0: return 18;
    case T_Q8_0: return 34;
    case T_Q4_K: return 144;
    case T_Q6_K: return 210;
    case T_IQ2_XXS: return 66;
    case T_IQ4_XS: return 136;
    case T_Q4_1: return 20;
    case T_Q5_0: return 22;
    case T_Q5_1: return 24;
    case T_Q5_K: return 176;
    case T_IQ4_NL: return 18;
    case T_IQ2_XS: return 74;
    case T_IQ2_S: return 82;
    case T_IQ3_XXS: return 98;
    case T_IQ3_S: return 110;
    case T_IQ1_S: return 50;
    case T_IQ1_M: return 56;
    case T_Q2_K: return 84;
    case T_Q3_K: return 110;
  }
  return 0;
}
__host__ __device__ inline int block_size(int t) {
  switch (t) {
    case T_Q4_0: case T_Q8_0: case T_Q4_1: case T_Q5_0: case T_Q5_1: case T_IQ4_NL: return 32;
  }
  return type_size(t) ? 256 : 0;
}
// the same for every type the standalone dequantize knows (today the same set)
__host__ __device__ inline int dequant_type_size(int t) { return type_size(t); }
__host__ __device__ inline int dequant_block_size(int t) { return type_size(t) ? block_size(t) : (dequant_type_size(t) ? 256 : 0); }
__host__ __device__ inline int64_t round_up(int64_t a, int64_t b) { return (a + b - 1) / b * b; }

// ---- typed stores -----------------------------------------------------------------
template <typename T> __device__ __forceinline__ T from_float(float f);
template <> __device__ __forceinline__ float from_float<float>(float f) { return f; }
template <> __device__ __forceinline__ __half from_float<__half>(float f) { return __float2half_rn(f); }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float f) { return __float2bfloat16_rn(f); }

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// ---- shared-memory addressing, mbarrier, bulk copy --------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// The same with a suspend-time hint: the thread may stay parked for up to `ns` nanoseconds (it is
// resumed as soon as the phase completes), instead of the much shorter default after which a
// waiting warp comes back to poll again -- polls that take issue slots from the warps that work.
__device__ __forceinline__ bool mbar_try_wait_parked(uint64_t* bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(ns)
      : "memory");
  return ok != 0;
}
// non-blocking probe of a phase (try_wait may park the thread; this never does)
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Every wait in this library is bounded in time: a poll may itself suspend the thread for a
// while, so the limit is counted in SM clock cycles (about a quarter of a second), after which
// the caller records a status word and leaves, so a lost completion cannot wedge the GPU.  A
// thread that gives up still has asynchronous work in flight (bulk copies into its shared memory,
// tensor-core instructions): it calls drain_pause() -- and the tensor-core kernel also waits for
// its last commit -- before its CTA may retire.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, long long limit_cycles = 500000000ll) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  do {
    if (mbar_try_wait_parked(bar, parity, 8000u)) return true;
  } while (clock64() - t0 < limit_cycles);
  return false;
}
// Pause of about a tenth of a millisecond, far longer than any bulk copy takes to land.
__device__ __forceinline__ void drain_pause() {
  for (int i = 0; i < 64; ++i) __nanosleep(2000);
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// 1-D bulk copy global -> shared of this CTA; src, dst and bytes multiples of 16.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst_smem)),
      "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

// Loads from shared memory through 32-bit shared-window addresses.  (A pointer that went through
// an integer cast loses its address space and the compiler falls back to generic 64-bit loads and
// address arithmetic; these helpers keep everything in the shared window.)  volatile: the loads
// stay behind the mbarrier wait that made the data visible.
__device__ __forceinline__ uint32_t lds32(uint32_t saddr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(saddr));
  return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t saddr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(saddr));
  return v;
}
__device__ __forceinline__ uint4 lds128s(uint32_t saddr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(saddr));
  return v;
}
__device__ __forceinline__ float lds_half_f32(uint32_t saddr) {   // one fp16 value, widened
  unsigned short h;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(h) : "r"(saddr));
  return __half2float(__ushort_as_half(h));
}
template <int N> __device__ __forceinline__ void lds_words_unaligned(uint32_t a, uint32_t (&w)[N]) {
  const uint32_t al = a & ~3u, sh = (a & 3u) * 8u;
  uint32_t r[N + 1];
#pragma unroll
  for (int i = 0; i <= N; ++i) r[i] = lds32(al + 4u * i);
#pragma unroll
  for (int i = 0; i < N; ++i) w[i] = __funnelshift_r(r[i], r[i + 1], sh);
}
// N consecutive 32-bit words starting at a shared address that is only 2-byte aligned: the N + 1
// aligned words that cover them, realigned with funnel shifts.
template <int N> __device__ __forceinline__ void lds_words_unaligned(const uint8_t* p, uint32_t (&w)[N]) {
  lds_words_unaligned<N>(smem_u32(p), w);
}
// 32-bit word from shared memory at an address that is only 2-byte aligned.
__device__ __forceinline__ uint32_t lds_u32_a2(const uint8_t* p) {
  uint32_t w[1];
  lds_words_unaligned<1>(p, w);
  return w[0];
}
__device__ __forceinline__ float lds_half_as_float(const uint8_t* p) {
  return __half2float(*reinterpret_cast<const __half*>(p));
}

// ---- packets of a gathered vector (tensor-parallel decode) ---------------------------------
// One element travels as ONE naturally aligned store that carries the value and the number of
// the launch that produced it: 32 bits {16-bit value, 16-bit tag} for f16 / bf16, 64 bits
// {f32 value, 32-bit tag} for f32.  A reader polls the word until the tag is the one it expects;
// the value then is that launch's, with no fence and no separate flag.  The poll is bounded.
template <typename T> __device__ __forceinline__ bool packet_read(const void* base, int64_t i, unsigned want, long long limit_cycles, float& out) {
  if (sizeof(T) == 2) {
    const uint32_t* p = static_cast<const uint32_t*>(base) + i;
    want &= 0xFFFFu;
    uint32_t v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    bool ok = (v >> 16) == want;
    if (!ok) {
      const long long t0 = clock64();
      do {
        asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
        ok = (v >> 16) == want;
      } while (!ok && clock64() - t0 < limit_cycles);
    }
    const unsigned short b = (unsigned short)(v & 0xFFFFu);
    out = to_float<T>(*reinterpret_cast<const T*>(&b));
    return ok;
  } else {
    const unsigned long long* p = static_cast<const unsigned long long*>(base) + i;
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    bool ok = (unsigned)(v >> 32) == want;
    if (!ok) {
      const long long t0 = clock64();
      do {
        asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
        ok = (unsigned)(v >> 32) == want;
      } while (!ok && clock64() - t0 < limit_cycles);
    }
    out = __uint_as_float((unsigned)(v & 0xFFFFFFFFull));
    return ok;
  }
}

// Programmatic dependent launch.  A kernel launched with launch_pdl() may become resident while
// the kernel before it in the stream is still running; pdl_wait() blocks until that kernel has
// completed and its writes are visible (it returns at once under a normal launch), and
// pdl_trigger() tells the runtime that the NEXT kernel in the stream may start launching.
// Rule used throughout: before pdl_wait() a kernel touches only memory no kernel writes
// (weights, codebooks) and its own shared memory.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
  return v;
}

// Host: launch with the programmatic-stream-serialization attribute (GGUF_B200_PDL=0 turns it off).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  static const bool enabled = [] {
    const char* v = getenv("GGUF_B200_PDL");
    return !(v && v[0] == '0');
  }();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = enabled ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

}  // namespace gguf_b200
